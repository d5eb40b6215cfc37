// What lies between a fused q/k/v projection and attention over the paged cache, in one pass per token:
//
//   1. optional RMS norm of the WHOLE query row and of the whole key row (all heads at once, one gain per
//      element; eps inside the root), in 32-bit;
//   2. optional rotary position encoding of queries and keys on the first `rot_dims` entries of every head
//      ("rotate half": entry i pairs with entry i + rot_dims / 2; the pair (u, v) at position p becomes
//      (u cos a - v sin a, v cos a + u sin a), a = p * freq[i]), positions and angles in 32-bit; the
//      frequencies come from the caller, who has applied whatever rescaling the model wants;
//   3. keys and values written into the request's pages, queries into a dense matrix, each head padded
//      with zeros from its own size up to the cache's head size (key size and value size may differ: the
//      cache and the attention kernels see one head size, the larger of the two rounded up to 16);
//      optionally each query head times a number of its own (a learned temperature: it reaches the scores through
//      the query), and each value head divided by its root mean square over its own entries (eps inside the root,
//      no gain), in 32-bit, so that the cache holds unit-RMS values;
//   4. optional per-head output gate: gate_out[t, h] = sigmoid(gate_in[t, h]) * gate_scale, 32-bit, which
//      the attention kernels multiply into a head's output.
//
// One block per token.  The step's tokens find their pages as everywhere: token -> request -> block table.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_prepare_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int n_heads, int n_kv_heads,
                         int qk_dim, int v_dim, int pad_dim, const float* __restrict__ q_gain,
                         const float* __restrict__ k_gain, float eps, const float* __restrict__ freq, int rot_dims,
                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ block_table, int max_blocks, T* __restrict__ k_cache,
                         T* __restrict__ v_cache, long long page_stride, int page_size, int num_pages, int write_cache,
                         T* __restrict__ q_out, int ld_q, const float* __restrict__ gate_in, int ld_gate,
                         float* __restrict__ gate_out, float gate_scale, const float* __restrict__ q_head_scale,
                         float v_unit_eps, int per_head_norm, float q_pos_coef, int q_pos_every, int* __restrict__ status) {
    __shared__ float scratch[32];
    extern __shared__ float cs[];                    // cos [rot_dims / 2], sin [rot_dims / 2], then 1 / rms of each value head,
    float* v_inv = cs + rot_dims;                    // then (per_head_norm) 1 / rms of each query head and each key head
    float* head_inv = v_inv + n_kv_heads;
    const int t = blockIdx.x;
    const int half = rot_dims / 2;
    const int pos = positions[t];                    // the step's index arrays were staged before the step
    if (freq)
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float a = (float)pos * freq[i];
            float s, c;
            sincosf(a, &s, &c);
            cs[i] = c;
            cs[half + i] = s;
        }
    pdl_wait();
    pdl_launch_dependents();
    const T* row = proj + (size_t)t * ld;
    const int nq = n_heads * qk_dim, nk = n_kv_heads * qk_dim, nv = n_kv_heads * v_dim;
    float q_inv = 1.0f, k_inv = 1.0f;
    // a factor on the whole query that grows with the position: 1 + coef * ln(floor((pos + 1) / every) + 1), in 32-bit
    const float q_pos_scale = q_pos_every > 0 ? 1.0f + q_pos_coef * logf((float)((pos + 1) / q_pos_every) + 1.0f) : 1.0f;
    if (per_head_norm) {                             // a warp a head: the query heads, then the key heads
        for (int g = threadIdx.x >> 5; g < n_heads + n_kv_heads; g += blockDim.x >> 5) {
            const int base = g < n_heads ? q_off + g * qk_dim : k_off + (g - n_heads) * qk_dim;
            float ss = 0.0f;
            for (int i = threadIdx.x & 31; i < qk_dim; i += 32) {
                const float x = to_f32(row[base + i]);
                ss = fmaf(x, x, ss);
            }
            ss = warp_sum(ss);
            if ((threadIdx.x & 31) == 0) head_inv[g] = 1.0f / sqrtf(ss / (float)qk_dim + eps);
        }
    }
    if (q_gain && !per_head_norm) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) {
            const float x = to_f32(row[q_off + i]);
            ss = fmaf(x, x, ss);
        }
        q_inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nq + eps);
    }
    if (k_gain && !per_head_norm) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const float x = to_f32(row[k_off + i]);
            ss = fmaf(x, x, ss);
        }
        k_inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nk + eps);
    }
    if (v_unit_eps > 0.0f)                           // a warp a value head
        for (int g = threadIdx.x >> 5; g < n_kv_heads; g += blockDim.x >> 5) {
            float ss = 0.0f;
            for (int i = threadIdx.x & 31; i < v_dim; i += 32) {
                const float x = to_f32(row[v_off + g * v_dim + i]);
                ss = fmaf(x, x, ss);
            }
            ss = warp_sum(ss);
            if ((threadIdx.x & 31) == 0) v_inv[g] = 1.0f / sqrtf(ss / (float)v_dim + v_unit_eps);
        }
    __syncthreads();                                 // cs and v_inv are complete (block_sum may not have run)

    // where this token's key and value go
    long long page_base = -1;
    if (write_cache) {
        const int s = token_seq[t];
        const int page = (pos >= 0 && pos / page_size < max_blocks) ? block_table[(size_t)s * max_blocks + pos / page_size] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && status) atomicOr(status, 8);
        } else {
            page_base = (long long)page * page_stride + (long long)(pos % page_size) * pad_dim;
        }
    }

    // one normed and turned entry of the query (which = 0) or the key (which = 1)
    auto turned = [&](int off, const float* gain, float inv, int head, int i) -> float {
        const int base = off + head * qk_dim;
        auto normed = [&](int j) { return to_f32(row[base + j]) * inv * (gain ? gain[head * qk_dim + j] : 1.0f); };
        if (!freq || i >= rot_dims) return normed(i);
        if (i < half) return normed(i) * cs[i] - normed(i + half) * cs[half + i];
        return normed(i) * cs[i - half] + normed(i - half) * cs[i];
    };

    for (int idx = threadIdx.x; idx < n_heads * pad_dim; idx += blockDim.x) {
        const int h = idx / pad_dim, i = idx % pad_dim;
        const float inv = per_head_norm ? head_inv[h] : q_inv;
        q_out[(size_t)t * ld_q + idx] =
            from_f32<T>(i < qk_dim ? turned(q_off, q_gain, inv, h, i) * (q_head_scale ? q_head_scale[h] : 1.0f) * q_pos_scale : 0.0f);
    }
    if (page_base >= 0) {
        for (int idx = threadIdx.x; idx < n_kv_heads * pad_dim; idx += blockDim.x) {
            const int g = idx / pad_dim, i = idx % pad_dim;
            const long long dst = page_base + (long long)g * page_size * pad_dim + i;
            k_cache[dst] = from_f32<T>(i < qk_dim ? turned(k_off, k_gain, per_head_norm ? head_inv[n_heads + g] : k_inv, g, i) : 0.0f);
            if (v_unit_eps > 0.0f) v_cache[dst] = from_f32<T>(i < v_dim ? to_f32(row[v_off + g * v_dim + i]) * v_inv[g] : 0.0f);
            else v_cache[dst] = i < v_dim ? row[v_off + g * v_dim + i] : from_f32<T>(0.0f);
        }
    }
    (void)nv;
    if (gate_out)
        for (int h = threadIdx.x; h < n_heads; h += blockDim.x)
            gate_out[(size_t)t * n_heads + h] = gate_scale / (1.0f + expf(-gate_in[(size_t)t * ld_gate + h]));
}

}  // namespace

// proj: [n_tokens, *] of dtype with pitch ld; queries start at column q_off (n_heads * qk_dim of them), keys at
// k_off (n_kv_heads * qk_dim), values at v_off (n_kv_heads * v_dim).  q_gain / k_gain: float32 or null (no norm).
// freq: float32 [rot_dims / 2] or null (no rotation).  The cache's head size is pad_dim >= max(qk_dim, v_dim).
// q_out: [n_tokens, n_heads * pad_dim] of dtype.  gate_in: float32 [n_tokens, >= n_heads] with pitch ld_gate, or null.
// q_head_scale: float32 [n_heads] or null; v_unit_eps > 0: value heads are divided by their root mean square.
// per_head_norm != 0: every query head and every key head is divided by its own root mean square over qk_dim (eps inside
// the root; the gains, [heads * qk_dim], may then be null) instead of the norm over the whole row.  q_pos_every > 0: the
// query at position p is multiplied by 1 + q_pos_coef * ln(floor((p + 1) / q_pos_every) + 1).
SANDY_API int sandy_attention_prepare_pos(const void* proj, int ld, int q_off, int k_off, int v_off, int n_tokens, int n_heads,
                                      int n_kv_heads, int qk_dim, int v_dim, int pad_dim, const float* q_gain,
                                      const float* k_gain, float eps, const float* freq, int rot_dims, const int* positions,
                                      const int* token_seq, const int* block_table, int max_blocks, void* k_cache,
                                      void* v_cache, long long page_stride, int page_size, int num_pages, int write_cache,
                                      void* q_out, int ld_q, const float* gate_in, int ld_gate, float* gate_out,
                                      float gate_scale, const float* q_head_scale, float v_unit_eps, int per_head_norm,
                                      float q_pos_coef, int q_pos_every, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!proj || !positions || !token_seq || !q_out || (write_cache && (!block_table || !k_cache || !v_cache)))
        return SANDY_ERR_ARGUMENT;
    if (pad_dim < qk_dim || pad_dim < v_dim || rot_dims < 0 || rot_dims > qk_dim || (rot_dims & 1) || (gate_out && !gate_in))
        return SANDY_ERR_UNSUPPORTED;
    const size_t smem = ((size_t)rot_dims + (size_t)n_kv_heads + (per_head_norm ? (size_t)(n_heads + n_kv_heads) : 0)) * sizeof(float);
    if (smem > 32 * 1024) return SANDY_ERR_UNSUPPORTED;
    if (dtype == SANDY_F32)
        return sandy_launch(attention_prepare_kernel<float>, dim3(n_tokens), dim3(THREADS), smem, stream, (const float*)proj,
                            ld, q_off, k_off, v_off, n_heads, n_kv_heads, qk_dim, v_dim, pad_dim, q_gain, k_gain, eps, freq,
                            rot_dims, positions, token_seq, block_table, max_blocks, (float*)k_cache, (float*)v_cache,
                            page_stride, page_size, num_pages, write_cache, (float*)q_out, ld_q, gate_in, ld_gate, gate_out,
                            gate_scale, q_head_scale, v_unit_eps, per_head_norm, q_pos_coef, q_pos_every, status);
    if (dtype == SANDY_BF16)
        return sandy_launch(attention_prepare_kernel<bf16>, dim3(n_tokens), dim3(THREADS), smem, stream, (const bf16*)proj,
                            ld, q_off, k_off, v_off, n_heads, n_kv_heads, qk_dim, v_dim, pad_dim, q_gain, k_gain, eps, freq,
                            rot_dims, positions, token_seq, block_table, max_blocks, (bf16*)k_cache, (bf16*)v_cache,
                            page_stride, page_size, num_pages, write_cache, (bf16*)q_out, ld_q, gate_in, ld_gate, gate_out,
                            gate_scale, q_head_scale, v_unit_eps, per_head_norm, q_pos_coef, q_pos_every, status);
    return SANDY_ERR_UNSUPPORTED;
}

// The same with the norms over whole rows and no factor by position.
SANDY_API int sandy_attention_prepare_ext(const void* proj, int ld, int q_off, int k_off, int v_off, int n_tokens, int n_heads,
                                      int n_kv_heads, int qk_dim, int v_dim, int pad_dim, const float* q_gain,
                                      const float* k_gain, float eps, const float* freq, int rot_dims, const int* positions,
                                      const int* token_seq, const int* block_table, int max_blocks, void* k_cache,
                                      void* v_cache, long long page_stride, int page_size, int num_pages, int write_cache,
                                      void* q_out, int ld_q, const float* gate_in, int ld_gate, float* gate_out,
                                      float gate_scale, const float* q_head_scale, float v_unit_eps, int dtype, int* status,
                                      cudaStream_t stream) {
    return sandy_attention_prepare_pos(proj, ld, q_off, k_off, v_off, n_tokens, n_heads, n_kv_heads, qk_dim, v_dim, pad_dim, q_gain,
                                       k_gain, eps, freq, rot_dims, positions, token_seq, block_table, max_blocks, k_cache, v_cache,
                                       page_stride, page_size, num_pages, write_cache, q_out, ld_q, gate_in, ld_gate, gate_out,
                                       gate_scale, q_head_scale, v_unit_eps, 0, 0.0f, 0, dtype, status, stream);
}

// The same without a factor per query head and with the values as projected.
SANDY_API int sandy_attention_prepare(const void* proj, int ld, int q_off, int k_off, int v_off, int n_tokens, int n_heads,
                                      int n_kv_heads, int qk_dim, int v_dim, int pad_dim, const float* q_gain,
                                      const float* k_gain, float eps, const float* freq, int rot_dims, const int* positions,
                                      const int* token_seq, const int* block_table, int max_blocks, void* k_cache,
                                      void* v_cache, long long page_stride, int page_size, int num_pages, int write_cache,
                                      void* q_out, int ld_q, const float* gate_in, int ld_gate, float* gate_out,
                                      float gate_scale, int dtype, int* status, cudaStream_t stream) {
    return sandy_attention_prepare_ext(proj, ld, q_off, k_off, v_off, n_tokens, n_heads, n_kv_heads, qk_dim, v_dim, pad_dim, q_gain,
                                       k_gain, eps, freq, rot_dims, positions, token_seq, block_table, max_blocks, k_cache, v_cache,
                                       page_stride, page_size, num_pages, write_cache, q_out, ld_q, gate_in, ld_gate, gate_out,
                                       gate_scale, nullptr, 0.0f, dtype, status, stream);
}
