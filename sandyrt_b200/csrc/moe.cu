// Routing of a mixture of experts, all on the device (a recorded step serves every routing):
//
//   sandy_moe_route    per token: logits z = router product + bias (32-bit); the `top` largest (ties: the lower
//                      expert first) are chosen, their weights are the softmax over the chosen logits alone.
//                      Entry t * top + j holds the j-th choice of token t.
//   sandy_moe_route_scored
//                      per token: scores s = sigmoid(z); choice scores c = s + correction; the experts form `n_groups`
//                      equal groups of neighbours, a group's score is the sum of its `group_rank` largest choice
//                      scores, and only experts of the `keep_groups` best groups can be chosen (ties: the lower group
//                      and the lower expert first); the `top` largest c among those are chosen; their weights are
//                      their s over the sum of the chosen s (+ norm_eps), times weight_scale.
//   sandy_moe_route_softmax
//                      per token: scores s = softmax(z) over all experts; the `top` largest s + correction are chosen;
//                      their weights are their s themselves (not renormalised unless asked).
//   sandy_moe_group    entries sorted by expert: group_start[e] .. group_start[e+1]-1 are expert e's slots;
//                      entry_of_slot and slot_of_entry are the two directions of the permutation.  Which slot of
//                      its expert an entry gets is not fixed from run to run; nothing depends on it, since every
//                      slot's row is computed on its own.
//   sandy_moe_gather   sorted[s] = x[token of slot s]: the tokens' rows in the order of the slots, for a product that
//                      wants every expert's rows one after another.
//   sandy_moe_combine  y[t] (+)= sum_j weight[t, j] * rows[slot_of_entry[t * top + j]], in 32-bit, j in order.
//   sandy_moe_combine_identity
//                      the same where the last experts are identities: their entries contribute weight * the token's
//                      own input row.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, int n_tokens, int n_experts,
                 int top, int* __restrict__ expert_of, float* __restrict__ weight_of) {
    extern __shared__ float z_all[];                 // [warps][n_experts]
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    float* z = z_all + (size_t)warp * n_experts;
    for (int e = lane; e < n_experts; e += 32) z[e] = logits[(size_t)t * ld + e] + (bias ? bias[e] : 0.0f);
    __syncwarp();
    float first = 0.0f, sum = 0.0f;
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; arg = e; }     // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = j;              // every logit NaN or -inf: any expert, weight below is NaN or 0
        if (j == 0) first = best;
        const float w = expf(best - first);
        sum += w;
        if (lane == 0) {
            expert_of[(size_t)t * top + j] = arg;
            weight_of[(size_t)t * top + j] = w;
            z[arg] = -INFINITY;
        }
        __syncwarp();
    }
    for (int j = lane; j < top; j += 32) weight_of[(size_t)t * top + j] /= sum;      // lane 0's writes are visible after the syncwarp
}

// A warp a token.  Shared memory per warp: choice scores [n_experts], plain scores [n_experts], group scores [n_groups].
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction, int n_tokens,
                        int n_experts, int top, int n_groups, int keep_groups, int group_rank, float weight_scale,
                        float norm_eps, int softmax_scores, int renormalize, int* __restrict__ expert_of,
                        float* __restrict__ weight_of) {
    extern __shared__ float route_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    float* c = route_smem + (size_t)warp * (2 * n_experts + n_groups);
    float* sc = c + n_experts;
    float* gs = sc + n_experts;
    float z_max = -INFINITY, z_sum = 1.0f;
    if (softmax_scores) {                            // s = softmax over all experts' logits
        for (int e = lane; e < n_experts; e += 32) z_max = fmaxf(z_max, logits[(size_t)t * ld + e]);
        z_max = warp_max(z_max);
        float part = 0.0f;
        for (int e = lane; e < n_experts; e += 32) part += expf(logits[(size_t)t * ld + e] - z_max);
        z_sum = warp_sum(part);
    }
    for (int e = lane; e < n_experts; e += 32) {
        const float z = logits[(size_t)t * ld + e];
        const float s = softmax_scores ? expf(z - z_max) / z_sum : 1.0f / (1.0f + expf(-z));
        sc[e] = s;
        c[e] = s + (correction ? correction[e] : 0.0f);
    }
    __syncwarp();
    if (n_groups > 1 && keep_groups < n_groups) {
        const int per = n_experts / n_groups;
        // a lane a group: the sum of its group_rank largest choice scores
        for (int g = lane; g < n_groups; g += 32) {
            float sum = 0.0f;
            for (int i = 0; i < per; i++) {          // an entry counts if fewer than group_rank entries are ahead of it
                const float v = c[g * per + i];
                int ahead = 0;
                for (int k = 0; k < per; k++) {
                    const float o = c[g * per + k];
                    if (o > v || (o == v && k < i)) ahead++;
                }
                if (ahead < group_rank) sum += v;
            }
            gs[g] = sum;
        }
        __syncwarp();
        // a lane a group again: a group is kept if fewer than keep_groups groups are ahead of it
        for (int g = lane; g < n_groups; g += 32) {
            int ahead = 0;
            const float v = gs[g];
            for (int k = 0; k < n_groups; k++) {
                const float o = gs[k];
                if (o > v || (o == v && k < g)) ahead++;
            }
            if (ahead >= keep_groups)
                for (int i = 0; i < per; i++) c[g * per + i] = -INFINITY;
        }
        __syncwarp();
    }
    float sum = 0.0f;
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = c[e];
            if (v > best) { best = v; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = j;              // nothing left to choose from (NaN logits): any expert
        const float w = sc[arg];
        sum += w;
        if (lane == 0) {
            expert_of[(size_t)t * top + j] = arg;
            weight_of[(size_t)t * top + j] = w;
            c[arg] = -INFINITY;
        }
        __syncwarp();
    }
    const float denom = renormalize ? sum + norm_eps : 1.0f;
    for (int j = lane; j < top; j += 32) weight_of[(size_t)t * top + j] = weight_of[(size_t)t * top + j] / denom * weight_scale;
}

__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ expert_of, int n_entries, int n_experts, int* __restrict__ group_start,
                 int* __restrict__ entry_of_slot, int* __restrict__ slot_of_entry) {
    extern __shared__ int counts[];                  // [n_experts] counts, then [n_experts] cursors
    int* cursor = counts + n_experts;
    pdl_wait();
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_entries; i += blockDim.x) {
        const int e = expert_of[i];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_experts; e++) {
            group_start[e] = at;
            cursor[e] = at;
            at += counts[e];
        }
        group_start[n_experts] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_entries; i += blockDim.x) {
        const int e = expert_of[i];
        if (e < 0 || e >= n_experts) continue;
        const int s = atomicAdd(&cursor[e], 1);
        entry_of_slot[s] = i;
        slot_of_entry[i] = s;
    }
}

template <typename V>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const V* __restrict__ x, long long ldx, const int* __restrict__ entry_of_slot, int top, V* __restrict__ out,
                  long long ldo, int n_slots, int cols) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long)n_slots * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long s = i / cols, c = i % cols;
        out[s * ldo + c] = x[(long long)(entry_of_slot[s] / top) * ldx + c];
    }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ rows, int ld_rows, const float* __restrict__ weight_of,
                   const int* __restrict__ slot_of_entry, int top, float* __restrict__ y, int ldy, int width, int add,
                   const int* __restrict__ expert_of, int n_real, const void* __restrict__ h, int ldh, int h_dtype) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < top; j++) {
            float v;
            if (expert_of && expert_of[(size_t)t * top + j] >= n_real) {      // an expert that hands its input on
                v = h_dtype == SANDY_BF16 ? to_f32(((const bf16*)h)[(size_t)t * ldh + c]) : ((const float*)h)[(size_t)t * ldh + c];
            } else {
                v = rows[(size_t)slot_of_entry[(size_t)t * top + j] * ld_rows + c];
            }
            acc = fmaf(weight_of[(size_t)t * top + j], v, acc);
        }
        float* dst = y + (size_t)t * ldy + c;
        *dst = add ? *dst + acc : acc;
    }
}

}  // namespace

// logits: float32 [n_tokens, >= n_experts] with pitch ld; bias float32 [n_experts] or null; 1 <= top <= n_experts <= 2048.
SANDY_API int sandy_moe_route(const float* logits, int ld, const float* bias, int n_tokens, int n_experts, int top,
                              int* expert_of, float* weight_of, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!logits || !expert_of || !weight_of) return SANDY_ERR_ARGUMENT;
    if (top < 1 || top > n_experts || n_experts > 2048) return SANDY_ERR_UNSUPPORTED;
    const int warps = 4;
    return sandy_launch(moe_route_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps),
                        (size_t)warps * n_experts * sizeof(float), stream, logits, ld, bias, n_tokens, n_experts, top, expert_of,
                        weight_of);
}

// logits: float32 [n_tokens, >= n_experts] with pitch ld; correction float32 [n_experts] or null; n_groups divides
// n_experts; 1 <= keep_groups <= n_groups; with n_groups 1 (or every group kept) the groups play no part.
SANDY_API int sandy_moe_route_scored(const float* logits, int ld, const float* correction, int n_tokens, int n_experts, int top,
                                     int n_groups, int keep_groups, int group_rank, float weight_scale, float norm_eps,
                                     int* expert_of, float* weight_of, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!logits || !expert_of || !weight_of) return SANDY_ERR_ARGUMENT;
    if (top < 1 || top > n_experts || n_experts > 2048 || n_groups < 1 || n_experts % n_groups || keep_groups < 1 ||
        keep_groups > n_groups || group_rank < 1 || top > (n_experts / n_groups) * keep_groups)
        return SANDY_ERR_UNSUPPORTED;
    const int warps = 4;
    return sandy_launch(moe_route_scored_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps),
                        (size_t)warps * (2 * n_experts + n_groups) * sizeof(float), stream, logits, ld, correction, n_tokens,
                        n_experts, top, n_groups, keep_groups, group_rank, weight_scale, norm_eps, 0, 1, expert_of, weight_of);
}

// Scores s = softmax over ALL experts' logits; the choice is by s + correction (ties: the lower expert first); the
// weights are the chosen experts' s themselves, times weight_scale, over their sum (+ norm_eps) only with renormalize.
SANDY_API int sandy_moe_route_softmax(const float* logits, int ld, const float* correction, int n_tokens, int n_experts, int top,
                                      float weight_scale, float norm_eps, int renormalize, int* expert_of, float* weight_of,
                                      cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!logits || !expert_of || !weight_of) return SANDY_ERR_ARGUMENT;
    if (top < 1 || top > n_experts || n_experts > 2048) return SANDY_ERR_UNSUPPORTED;
    const int warps = 4;
    return sandy_launch(moe_route_scored_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps),
                        (size_t)warps * (2 * n_experts + 1) * sizeof(float), stream, logits, ld, correction, n_tokens, n_experts,
                        top, 1, 1, 1, weight_scale, norm_eps, 1, renormalize, expert_of, weight_of);
}

SANDY_API int sandy_moe_group(const int* expert_of, int n_entries, int n_experts, int* group_start, int* entry_of_slot,
                              int* slot_of_entry, cudaStream_t stream) {
    if (!expert_of || !group_start || !entry_of_slot || !slot_of_entry) return SANDY_ERR_ARGUMENT;
    if (n_experts < 1 || n_experts > 4096) return SANDY_ERR_UNSUPPORTED;
    return sandy_launch(moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * n_experts * sizeof(int), stream, expert_of,
                        n_entries, n_experts, group_start, entry_of_slot, slot_of_entry);
}

// rows: float32 [n_tokens * top, width] by slot; y: float32 [n_tokens, width]; add != 0 adds to y, else writes it.
SANDY_API int sandy_moe_combine(const float* rows, int ld_rows, const float* weight_of, const int* slot_of_entry, int n_tokens,
                                int top, float* y, int ldy, int width, int add, cudaStream_t stream) {
    if (n_tokens == 0 || width == 0) return SANDY_OK;
    if (!rows || !weight_of || !slot_of_entry || !y) return SANDY_ERR_ARGUMENT;
    return sandy_launch(moe_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, rows, ld_rows, weight_of, slot_of_entry, top,
                        y, ldy, width, add, (const int*)nullptr, 0, (const void*)nullptr, 0, SANDY_F32);
}

// The same where the experts from n_real on have no matrices and hand their input on: an entry whose expert_of is
// n_real or more contributes weight * h[t] (h [n_tokens, width] of h_dtype) instead of a computed row.
SANDY_API int sandy_moe_combine_identity(const float* rows, int ld_rows, const float* weight_of, const int* slot_of_entry,
                                         const int* expert_of, int n_real, const void* h, int ldh, int h_dtype, int n_tokens,
                                         int top, float* y, int ldy, int width, int add, cudaStream_t stream) {
    if (n_tokens == 0 || width == 0) return SANDY_OK;
    if (!rows || !weight_of || !slot_of_entry || !y || !expert_of || !h) return SANDY_ERR_ARGUMENT;
    if (h_dtype != SANDY_F32 && h_dtype != SANDY_BF16) return SANDY_ERR_UNSUPPORTED;
    return sandy_launch(moe_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, rows, ld_rows, weight_of, slot_of_entry, top,
                        y, ldy, width, add, expert_of, n_real, h, ldh, h_dtype);
}

// x: [tokens, bytes_per_row] and out: [n_slots, bytes_per_row] as raw bytes with pitches in bytes; pieces of 16 bytes
// where everything is aligned so, else of 2.
SANDY_API int sandy_moe_gather(const void* x, long long pitch_x, const int* entry_of_slot, int top, void* out, long long pitch_out,
                               int n_slots, int bytes_per_row, cudaStream_t stream) {
    if (n_slots == 0 || bytes_per_row == 0) return SANDY_OK;
    if (!x || !entry_of_slot || !out || top < 1) return SANDY_ERR_ARGUMENT;
    const bool wide = !(bytes_per_row % 16) && !(pitch_x % 16) && !(pitch_out % 16) && !((uintptr_t)x & 15) && !((uintptr_t)out & 15);
    const int unit = wide ? 16 : 2;
    if (bytes_per_row % unit || pitch_x % unit || pitch_out % unit) return SANDY_ERR_UNSUPPORTED;
    const long long n = (long long)n_slots * (bytes_per_row / unit);
    long long blocks = (n + 255) / 256;
    const long long cap = (long long)sandy_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (wide)
        return sandy_launch(moe_gather_kernel<uint4>, dim3((unsigned)blocks), dim3(256), 0, stream, (const uint4*)x, pitch_x / 16,
                            entry_of_slot, top, (uint4*)out, pitch_out / 16, n_slots, bytes_per_row / 16);
    return sandy_launch(moe_gather_kernel<unsigned short>, dim3((unsigned)blocks), dim3(256), 0, stream, (const unsigned short*)x,
                        pitch_x / 2, entry_of_slot, top, (unsigned short*)out, pitch_out / 2, n_slots, bytes_per_row / 2);
}
