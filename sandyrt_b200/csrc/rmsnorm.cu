// RMS norm over the last dimension, statistics in 32-bit, in three forms:
//
//   sandy_rmsnorm        out[r] = x[rows[r]] * rsqrt(mean(x^2) + eps) * gain        (a norm in front of a sublayer)
//   sandy_rmsnorm_add    x[r]  += mult * y[r] * rsqrt(mean(y^2) + eps) * gain       (a norm behind a sublayer: the
//                                                                                    branch is normed, scaled and
//                                                                                    added to the float32 stream)
//   sandy_head_norm_gate out[t, h, :] = o[t, h, :] * rsqrt(mean_over_the_head(o^2) + eps) * gain * act(gate[t, h, :]) * scale
//                                                                                   (the read-out of a recurrent
//                                                                                    mixer: a norm per head, then
//                                                                                    an output gate)
//
//   sandy_rmsnorm_shift  h[t] = norm(x[t]) * gain;  out[t] = h[t] + (h[t-1] - h[t]) * mix                (token shift: what a
//                                                                                    mixer reads leans towards the
//                                                                                    token before; the h before a
//                                                                                    request's first token of the
//                                                                                    step is its state row, zeros at
//                                                                                    its very first token)
//   sandy_rmsnorm_keep   state[slot of s] = norm(x[last token of s]) * gain          for requests with several tokens
//
// The mean is over the row (or the head) with eps inside the root.  The input is float32 (the residual
// stream, a branch, a recurrence's read-out), the gain float32 or absent, sums are float32; only the
// result is rounded, once, to the output's type.
//
// A row belongs to one warp and stays in its registers between the reduction and the scaling (rows up
// to 4,096 wide; wider rows are read twice).  A block holds eight rows.
#include "common.cuh"

namespace {

constexpr int ROWS_PER_BLOCK = 8;
constexpr int MAX_ROUNDS = 32;         // rows up to 32 * 128 elements stay in registers

__device__ __forceinline__ float act_gate(float z, int act) {
    const float s = 1.0f / (1.0f + expf(-z));
    return act == 1 ? z * s : s;       // 1: silu, otherwise sigmoid
}

// mode 0: out = norm(x[rows]) (TO);  mode 1: xio += mult * norm(x) (float)
template <typename TO, int NV, int MODE>
__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
rmsnorm_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gain, TO* __restrict__ out, int ldo,
               const int* __restrict__ rows, int n_rows, int width, float eps, float mult) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + warp;
    // the gain is a weight, which no kernel writes: asked for before the wait for the kernel that produces x
    float g[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * 32 + lane;
        g[i] = (gain && e < width) ? gain[e] : 1.0f;
    }
    pdl_wait();
    pdl_launch_dependents();
    if (r >= n_rows) return;
    const float* row = x + (size_t)(rows ? rows[r] : r) * ldx;
    float v[NV];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * 32 + lane;
        v[i] = e < width ? row[e] : 0.0f;
        ss = fmaf(v[i], v[i], ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    TO* orow = out + (size_t)r * ldo;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * 32 + lane;
        if (e < width) {
            const float y = v[i] * inv * g[i];
            if (MODE == 0) orow[e] = from_f32<TO>(y);
            else orow[e] = from_f32<TO>(to_f32(orow[e]) + mult * y);
        }
    }
}

// rows of any width: two passes over global memory, a block per row
template <typename TO, int MODE>
__global__ void __launch_bounds__(256)
rmsnorm_wide_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gain, TO* __restrict__ out, int ldo,
                    const int* __restrict__ rows, int width, float eps, float mult) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const float* row = x + (size_t)(rows ? rows[r] : r) * ldx;
    float ss = 0.0f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) ss = fmaf(row[e], row[e], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    TO* orow = out + (size_t)r * ldo;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float y = row[e] * inv * (gain ? gain[e] : 1.0f);
        if (MODE == 0) orow[e] = from_f32<TO>(y);
        else orow[e] = from_f32<TO>(to_f32(orow[e]) + mult * y);
    }
}

template <typename TO, int MODE>
int launch(const float* x, int ldx, const float* gain, TO* out, int ldo, const int* rows, int n_rows, int width, float eps,
           float mult, cudaStream_t stream) {
    const dim3 grid((n_rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK), block(ROWS_PER_BLOCK * 32);
#define CASE(NV)                                                                                                        \
    if (width <= 32 * NV)                                                                                               \
        return sandy_launch(rmsnorm_kernel<TO, NV, MODE>, grid, block, 0, stream, x, ldx, gain, out, ldo, rows, n_rows, \
                            width, eps, mult)
    CASE(2); CASE(4); CASE(8); CASE(12); CASE(16); CASE(24); CASE(MAX_ROUNDS);
#undef CASE
    return sandy_launch(rmsnorm_wide_kernel<TO, MODE>, dim3(n_rows), dim3(256), 0, stream, x, ldx, gain, out, ldo, rows,
                        width, eps, mult);
}

// Token shift behind the norm, a block per token.  h of the token before is recomputed from its row of the stream
// (same sums in the same order as that token's own block forms them), or read from the request's state row for the
// first token of the request in this step.  A request with ONE token in the step also writes its h into the state
// here: its block is the row's only reader and writer.  Requests with more tokens leave that to keep_last_kernel,
// which runs behind this one, so that no block writes a row another block of the same launch reads.
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_shift_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gain, const float* __restrict__ mix,
                     float* __restrict__ state, long long state_stride, const int* __restrict__ token_seq,
                     const int* __restrict__ q_start, const int* __restrict__ seq_slots, TO* __restrict__ out, int ldo,
                     int width, float eps) {
    __shared__ float scratch[32], scratch_prev[32];
    const int t = blockIdx.x;
    const int s = token_seq[t];                      // the step's index arrays were staged before the step
    const int first = q_start[s], last = q_start[s + 1] - 1;
    float* srow = state + (long long)seq_slots[s] * state_stride;
    pdl_wait();
    pdl_launch_dependents();
    const float* row = x + (size_t)t * ldx;
    const float* prow = x + (size_t)(t > first ? t - 1 : t) * ldx;
    float ss = 0.0f, sp = 0.0f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        ss = fmaf(row[e], row[e], ss);
        sp = fmaf(prow[e], prow[e], sp);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    const float inv_prev = 1.0f / sqrtf(block_sum(sp, scratch_prev) / (float)width + eps);
    TO* orow = out + (size_t)t * ldo;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float g = gain ? gain[e] : 1.0f;
        const float h = row[e] * inv * g;
        const float before = t > first ? prow[e] * inv_prev * g : srow[e];
        orow[e] = from_f32<TO>(h + (before - h) * mix[e]);
        if (first == last) srow[e] = h;
    }
}

// The same with the rows in registers: NV rounds of the block's threads cover the width, weights are asked for before
// the wait for the kernel that produces x, every row is read once, and the second sum is formed only where the
// token before is in the step.  Sums run in the order of the kernel above.
template <typename TO, int NV>
__global__ void __launch_bounds__(256)
rmsnorm_shift_reg_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gain, const float* __restrict__ mix,
                         float* __restrict__ state, long long state_stride, const int* __restrict__ token_seq,
                         const int* __restrict__ q_start, const int* __restrict__ seq_slots, TO* __restrict__ out, int ldo,
                         int width, float eps) {
    __shared__ float scratch[32], scratch_prev[32];
    const int t = blockIdx.x;
    const int s = token_seq[t];
    const int first = q_start[s], last = q_start[s + 1] - 1;
    float* srow = state + (long long)seq_slots[s] * state_stride;
    const bool inside = t > first;                   // the token before is a row of this step
    float g[NV], m[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * blockDim.x + threadIdx.x;
        g[i] = (gain && e < width) ? gain[e] : 1.0f;
        m[i] = e < width ? mix[e] : 0.0f;
    }
    pdl_wait();
    pdl_launch_dependents();
    const float* row = x + (size_t)t * ldx;
    const float* prow = inside ? row - ldx : srow;
    float v[NV], p[NV];
    float ss = 0.0f, sp = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * blockDim.x + threadIdx.x;
        v[i] = e < width ? row[e] : 0.0f;
        p[i] = e < width ? prow[e] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < NV; i++) {
        ss = fmaf(v[i], v[i], ss);
        sp = fmaf(p[i], p[i], sp);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    const float inv_prev = inside ? 1.0f / sqrtf(block_sum(sp, scratch_prev) / (float)width + eps) : 0.0f;
    TO* orow = out + (size_t)t * ldo;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * blockDim.x + threadIdx.x;
        if (e < width) {
            const float h = v[i] * inv * g[i];
            const float before = inside ? p[i] * inv_prev * g[i] : p[i];
            orow[e] = from_f32<TO>(h + (before - h) * m[i]);
            if (first == last) srow[e] = h;
        }
    }
}

template <typename TO>
int launch_shift(const float* x, int ldx, const float* gain, const float* mix, float* state, long long state_stride,
                 const int* token_seq, const int* q_start, const int* seq_slots, TO* out, int ldo, int n_tokens, int width,
                 float eps, cudaStream_t stream) {
    const int threads = width >= 1024 ? 256 : 128;
#define CASE(NV)                                                                                                          \
    if (width <= threads * NV)                                                                                            \
        return sandy_launch(rmsnorm_shift_reg_kernel<TO, NV>, dim3(n_tokens), dim3(threads), 0, stream, x, ldx, gain, mix, \
                            state, state_stride, token_seq, q_start, seq_slots, out, ldo, width, eps)
    CASE(2); CASE(4); CASE(6); CASE(8); CASE(16);
#undef CASE
    return sandy_launch(rmsnorm_shift_kernel<TO>, dim3(n_tokens), dim3(threads), 0, stream, x, ldx, gain, mix, state,
                        state_stride, token_seq, q_start, seq_slots, out, ldo, width, eps);
}

// A block per request of the step; requests with one token were served by the kernel above.
__global__ void __launch_bounds__(256)
keep_last_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gain, float* __restrict__ state,
                 long long state_stride, const int* __restrict__ q_start, const int* __restrict__ seq_slots, int width,
                 float eps) {
    __shared__ float scratch[32];
    const int s = blockIdx.x;
    const int first = q_start[s], last = q_start[s + 1] - 1;
    pdl_wait();
    pdl_launch_dependents();
    if (last <= first) return;
    const float* row = x + (size_t)last * ldx;
    float ss = 0.0f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) ss = fmaf(row[e], row[e], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    float* srow = state + (long long)seq_slots[s] * state_stride;
    for (int e = threadIdx.x; e < width; e += blockDim.x) srow[e] = row[e] * inv * (gain ? gain[e] : 1.0f);
}

// One warp per (token, head).  gain_stride: 0 when all heads share one gain of `dim` entries, `dim` when
// every head has its own.  The head's values stay in registers (heads up to 512 wide).
template <typename TG, typename TO, int NV>
__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
head_norm_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gain, int gain_stride,
                      const TG* __restrict__ gate, int ldg, TO* __restrict__ out, int ld_out, int n_tokens, int n_heads,
                      int dim, float eps, int act, float scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * ROWS_PER_BLOCK + warp;
    const int t = (int)(pair / n_heads), h = (int)(pair % n_heads);
    float g[NV];
    const bool live = pair < (long long)n_tokens * n_heads;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * 32 + lane;
        g[i] = (live && gain && e < dim) ? gain[(size_t)h * gain_stride + e] : 1.0f;
    }
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    const float* src = o + (size_t)t * ldo + (size_t)h * dim;
    float v[NV];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * 32 + lane;
        v[i] = e < dim ? src[e] : 0.0f;
        ss = fmaf(v[i], v[i], ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = i * 32 + lane;
        if (e < dim) {
            float y = v[i] * inv * g[i] * scale;
            if (gate) y *= act_gate(to_f32(gate[(size_t)t * ldg + (size_t)h * dim + e]), act);
            out[(size_t)t * ld_out + (size_t)h * dim + e] = from_f32<TO>(y);
        }
    }
}

template <typename TG, typename TO>
int launch_head(const float* o, int ldo, const float* gain, int gain_stride, const TG* gate, int ldg, TO* out, int ld_out,
                int n_tokens, int n_heads, int dim, float eps, int act, float scale, cudaStream_t stream) {
    const long long pairs = (long long)n_tokens * n_heads;
    const dim3 grid((unsigned)((pairs + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK)), block(ROWS_PER_BLOCK * 32);
#define CASE(NV)                                                                                                         \
    if (dim <= 32 * NV)                                                                                                  \
        return sandy_launch(head_norm_gate_kernel<TG, TO, NV>, grid, block, 0, stream, o, ldo, gain, gain_stride, gate,  \
                            ldg, out, ld_out, n_tokens, n_heads, dim, eps, act, scale)
    CASE(1); CASE(2); CASE(4); CASE(8); CASE(16);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}

}  // namespace

// x: float32 rows with pitch ldx; gain: float32 [width] or null; out: [n_rows, width] with pitch ldo;
// rows: int32 [n_rows] or null (output row r is the norm of input row rows[r]).
SANDY_API int sandy_rmsnorm(const float* x, int ldx, const float* gain, void* out, int ldo, const int* rows, int n_rows,
                            int width, float eps, int out_dtype, cudaStream_t stream) {
    if (n_rows == 0) return SANDY_OK;
    if (!x || !out || width <= 0) return SANDY_ERR_ARGUMENT;
    if (out_dtype == SANDY_F32) return launch<float, 0>(x, ldx, gain, (float*)out, ldo, rows, n_rows, width, eps, 1.0f, stream);
    if (out_dtype == SANDY_BF16) return launch<bf16, 0>(x, ldx, gain, (bf16*)out, ldo, rows, n_rows, width, eps, 1.0f, stream);
    return SANDY_ERR_UNSUPPORTED;
}

// x[r] += mult * norm(y[r]) * gain, both float32.
SANDY_API int sandy_rmsnorm_add(const float* y, int ldy, const float* gain, float* x, int ldx, int n_rows, int width,
                                float eps, float mult, cudaStream_t stream) {
    if (n_rows == 0) return SANDY_OK;
    if (!x || !y || width <= 0) return SANDY_ERR_ARGUMENT;
    return launch<float, 1>(y, ldy, gain, x, ldx, nullptr, n_rows, width, eps, mult, stream);
}

// o: float32 [n_tokens, n_heads * dim] (pitch ldo); gate: [n_tokens, n_heads * dim] of gate_dtype (pitch ldg) or
// null; act 0 sigmoid, 1 silu; out: [n_tokens, n_heads * dim] of out_dtype (pitch ld_out).
SANDY_API int sandy_head_norm_gate(const float* o, int ldo, const float* gain, int gain_stride, const void* gate, int ldg,
                                   int gate_dtype, void* out, int ld_out, int out_dtype, int n_tokens, int n_heads, int dim,
                                   float eps, int act, float scale, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!o || !out || dim <= 0 || n_heads <= 0) return SANDY_ERR_ARGUMENT;
#define CASE(DG, DO, TG, TO)                                                                                             \
    if (gate_dtype == DG && out_dtype == DO)                                                                             \
        return launch_head<TG, TO>(o, ldo, gain, gain_stride, (const TG*)gate, ldg, (TO*)out, ld_out, n_tokens, n_heads, \
                                   dim, eps, act, scale, stream)
    CASE(SANDY_F32, SANDY_F32, float, float);
    CASE(SANDY_BF16, SANDY_BF16, bf16, bf16);
    CASE(SANDY_F32, SANDY_BF16, float, bf16);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}

// x: float32 [n_tokens, width] (pitch ldx); gain: float32 [width] or null; mix: float32 [width]; state: float32 rows of
// `state_stride` floats, one per state slot, the first `width` of which hold the request's last h; out: [n_tokens,
// width] of out_dtype.  token_seq [n_tokens], q_start [n_seqs + 1], seq_slots [n_seqs]: the step's index arrays.
SANDY_API int sandy_rmsnorm_shift(const float* x, int ldx, const float* gain, const float* mix, float* state,
                                  long long state_stride, const int* token_seq, const int* q_start, const int* seq_slots,
                                  void* out, int ldo, int n_tokens, int width, float eps, int out_dtype, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!x || !mix || !state || !token_seq || !q_start || !seq_slots || !out || width <= 0 || state_stride < width)
        return SANDY_ERR_ARGUMENT;
    if (out_dtype == SANDY_F32)
        return launch_shift(x, ldx, gain, mix, state, state_stride, token_seq, q_start, seq_slots, (float*)out, ldo, n_tokens,
                            width, eps, stream);
    if (out_dtype == SANDY_BF16)
        return launch_shift(x, ldx, gain, mix, state, state_stride, token_seq, q_start, seq_slots, (bf16*)out, ldo, n_tokens,
                            width, eps, stream);
    return SANDY_ERR_UNSUPPORTED;
}

// Runs behind sandy_rmsnorm_shift in steps that hold a request with more than one token.
SANDY_API int sandy_rmsnorm_keep(const float* x, int ldx, const float* gain, float* state, long long state_stride,
                                 const int* q_start, const int* seq_slots, int n_seqs, int width, float eps,
                                 cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!x || !state || !q_start || !seq_slots || width <= 0 || state_stride < width) return SANDY_ERR_ARGUMENT;
    return sandy_launch(keep_last_kernel, dim3(n_seqs), dim3(width >= 1024 ? 256 : 128), 0, stream, x, ldx, gain, state,
                        state_stride, q_start, seq_slots, width, eps);
}
