// Attention of single tokens over the paged cache where MANY query heads read ONE key/value head (bfloat16):
// the query heads of a group are the rows of the tensor-core instruction.
//
// Where attention runs over a latent, or with few key/value heads, all query heads of a group walk the same keys.
// The kernels of attention_decode*.cu take one (token, head) pair a block and read those keys once per head; here a
// block takes up to sixteen heads of one group at once: S = Q K^T with the heads as the sixteen rows of mma.sync
// m16n8k16 (nothing padded when a group has sixteen heads), the softmax row by row in the accumulator's registers,
// O += P V with P taken from those registers as the next product's A fragment.  Keys are fetched once per sixteen
// heads, and a head's arithmetic is one row of products the tensor cores do anyway.
//
// Block (split, group x row tile, token), four warps.  The token's visible keys are cut into groups of 16 counted
// from its first visible key; a split takes a run of groups, its warps every fourth group of the run, each at its own
// pace: 16-byte cp.async copies into a stage of its own (two stages: one being multiplied, one on its way; rows outside
// the range or without a page are zero-filled, so a poisoned slot never meets a zero of P), ldmatrix for the keys,
// ldmatrix.trans for the values.  Where keys and values are one plane (the cache's values are its keys) a group is
// fetched once and read twice.  The warps' running maxima, sums and accumulators meet in shared memory; with one split
// the block finishes the rows (sink into the denominator, the per-head output factor, division) and writes them;
// with more, every block leaves its partial rows in a scratch and a second kernel adds them in the splits' order.
// Formula, sink and output factor as in attention.cu; scores, softmax and sums in 32-bit, base 2 exponentials, P
// rounded to bfloat16 for the product (the row sum is taken before rounding).  Head sizes: multiples of 16 up to 128.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int GROUP = 16;                  // keys a warp multiplies at a time
constexpr int ROWS = 16;                   // query heads a block takes
constexpr int STAGES = 2;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4_t(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// A block's partial rows in the scratch: [ROWS][D + 2] floats: the accumulator, then the maximum and the sum.
template <int D>
__global__ void __launch_bounds__(WARPS * 32)
decode_shared_kernel(const bf16* __restrict__ q, int ld_q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                     long long page_stride, const int* __restrict__ block_table, int max_blocks,
                     const int* __restrict__ token_seq, const int* __restrict__ positions, bf16* __restrict__ out, int ld_out,
                     int n_heads, int n_kv_heads, int page_size, float scale, int window, float softcap, int chunk, int splits,
                     int num_pages, const float* __restrict__ sink, const float* __restrict__ out_gate,
                     const float* __restrict__ dist_bias, int n_dist, float* __restrict__ scratch, int* __restrict__ status) {
    constexpr int PITCH = D + 8;                       // elements: ldmatrix rows fall on different banks
    constexpr int PIECES = D / 8;                      // 16-byte pieces of a key row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const bool one_plane = k_cache == v_cache;
    const int planes = one_plane ? 1 : 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int t = blockIdx.z, split = blockIdx.x;
    const int group_heads = n_heads / n_kv_heads, row_tiles = (group_heads + ROWS - 1) / ROWS;
    const int kvh = blockIdx.y / row_tiles, row_tile = blockIdx.y % row_tiles;
    const int first_head = kvh * group_heads + row_tile * ROWS;
    const int valid_rows = min(ROWS, group_heads - row_tile * ROWS);

    pdl_wait();
    pdl_launch_dependents();
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_seq[t] * max_blocks;
    int lo = window > 0 ? max(0, pos + 1 - window) : 0;
    if (chunk > 0) lo = max(lo, pos - pos % chunk);          // a query sees the keys of its own chunk of positions
    const int n_groups = (pos + 1 - lo + GROUP - 1) / GROUP;
    const int per_split = (n_groups + splits - 1) / splits;
    const int g_begin = split * per_split, g_end = min(n_groups, g_begin + per_split);

    // this lane's pieces of the query rows, as the A fragments of S = Q K^T
    unsigned qa[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int row = gq + (i & 1) * 8, col = kk * 16 + tq * 2 + (i >> 1) * 8;
            qa[kk][i] = row < valid_rows ? *reinterpret_cast<const unsigned*>(q + (size_t)t * ld_q + (size_t)(first_head + row) * D + col) : 0u;
        }
    }
    bf16* stage = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * STAGES * planes * GROUP * PITCH;
    auto fetch = [&](int g, int st) {
        bf16* ks = stage + (size_t)st * planes * GROUP * PITCH;
#pragma unroll
        for (int i = 0; i < (GROUP * PIECES + 31) / 32; i++) {
            const int c = lane + 32 * i;
            if (c < GROUP * PIECES) {
                const int r = c / PIECES, piece = c % PIECES;
                const int key = lo + g * GROUP + r;
                long long src = -1;
                if (key <= pos && key / page_size < max_blocks) {
                    const int page = table[key / page_size];
                    if (page >= 0 && page < num_pages)
                        src = (long long)page * page_stride + ((long long)kvh * page_size + key % page_size) * D + piece * 8;
                    else if (status) atomicOr(status, 16);
                }
                cp16(ks + r * PITCH + piece * 8, src >= 0 ? (const void*)(k_cache + src) : (const void*)k_cache, src >= 0);
                if (!one_plane)
                    cp16(ks + GROUP * PITCH + r * PITCH + piece * 8, src >= 0 ? (const void*)(v_cache + src) : (const void*)v_cache, src >= 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    const float s2 = scale * LOG2E;
    const float cap2 = softcap * LOG2E, over_cap = softcap > 0.0f ? scale / softcap : 0.0f;      // capped: cap tanh(s scale / cap)
    int g = g_begin + warp, st = 0;
    if (g < g_end) fetch(g, 0);
    for (; g < g_end; g += WARPS, st ^= 1) {
        if (g + WARPS < g_end) {
            fetch(g + WARPS, st ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        const bf16* ks = stage + (size_t)st * planes * GROUP * PITCH;
        const bf16* vs = one_plane ? ks : ks + GROUP * PITCH;
        float s[2][4] = {};
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
            unsigned b[4];
            ldsm4(b, ks + ((lane & 7) + (lane >> 4) * 8) * PITCH + kk * 16 + ((lane >> 3) & 1) * 8);
            mma16816(s[0], qa[kk], b[0], b[1]);
            mma16816(s[1], qa[kk], b[2], b[3]);
        }
        // s[nt][0..1]: row gq, keys nt * 8 + tq * 2 (+ 1); s[nt][2..3]: row gq + 8
        const int key0 = lo + g * GROUP;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int key = key0 + nt * 8 + tq * 2 + (j & 1);
                float sc = softcap > 0.0f ? cap2 * tanh_fast(s[nt][j] * over_cap) : s[nt][j] * s2;
                if (dist_bias) {                               // a learned bias by distance, this row's head
                    const int hd = min(first_head + gq + (j >> 1) * 8, n_heads - 1);
                    sc = fmaf(__ldg(dist_bias + (size_t)hd * n_dist + min(max(pos - key, 0), n_dist - 1)), LOG2E, sc);
                }
                s[nt][j] = key <= pos ? sc : -INFINITY;
            }
        unsigned pa[4];
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const float mx = quad_max(fmaxf(fmaxf(s[0][half * 2], s[0][half * 2 + 1]), fmaxf(s[1][half * 2], s[1][half * 2 + 1])));
            const float m_new = fmaxf(m[half], mx);            // finite: a group holds at least one visible key
            const float corr = exp2f(m[half] - m_new);
            m[half] = m_new;
            const float p00 = exp2f(s[0][half * 2] - m_new), p01 = exp2f(s[0][half * 2 + 1] - m_new);
            const float p10 = exp2f(s[1][half * 2] - m_new), p11 = exp2f(s[1][half * 2 + 1] - m_new);
            l[half] = l[half] * corr + (p00 + p01 + p10 + p11);
#pragma unroll
            for (int i = 0; i < D / 8; i++) {
                acc[i][half * 2] *= corr;
                acc[i][half * 2 + 1] *= corr;
            }
            pa[half] = pack_bf16(p00, p01);                    // keys 0..7 of the group: k 0..7 of the next product
            pa[2 + half] = pack_bf16(p10, p11);                // keys 8..15
        }
#pragma unroll
        for (int i = 0; i < D / 16; i++) {
            unsigned b[4];
            ldsm4_t(b, vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + i * 16 + (lane >> 4) * 8);
            mma16816(acc[2 * i], pa, b[0], b[1]);
            mma16816(acc[2 * i + 1], pa, b[2], b[3]);
        }
        __syncwarp();                                          // the stage may be filled again
    }
    l[0] = quad_sum(l[0]);
    l[1] = quad_sum(l[1]);

    // the four warps' rows meet in shared memory: per warp [ROWS][D] sums, then [ROWS] maxima, [ROWS] sums
    __syncthreads();
    float* meet = reinterpret_cast<float*>(smem_raw);
    float* mine = meet + (size_t)warp * ROWS * (D + 2);
#pragma unroll
    for (int i = 0; i < D / 8; i++) {
        *reinterpret_cast<float2*>(mine + gq * D + i * 8 + tq * 2) = make_float2(acc[i][0], acc[i][1]);
        *reinterpret_cast<float2*>(mine + (gq + 8) * D + i * 8 + tq * 2) = make_float2(acc[i][2], acc[i][3]);
    }
    if (tq == 0) {
        mine[ROWS * D + gq] = m[0];
        mine[ROWS * D + gq + 8] = m[1];
        mine[ROWS * D + ROWS + gq] = l[0];
        mine[ROWS * D + ROWS + gq + 8] = l[1];
    }
    __syncthreads();
    float* part = scratch ? scratch + (((size_t)t * gridDim.y + blockIdx.y) * splits + split) * ROWS * (D + 2) : nullptr;
    for (int idx = threadIdx.x; idx < ROWS * D; idx += WARPS * 32) {
        const int row = idx / D, col = idx % D;
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; w++) big = fmaxf(big, meet[(size_t)w * ROWS * (D + 2) + ROWS * D + row]);
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) {
            const float* o = meet + (size_t)w * ROWS * (D + 2);
            const float mw = o[ROWS * D + row];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - big);
            num = fmaf(f, o[row * D + col], num);
            den = fmaf(f, o[ROWS * D + ROWS + row], den);
        }
        if (splits > 1) {
            part[row * (D + 2) + col] = num;
            if (col == 0) {
                part[row * (D + 2) + D] = big;
                part[row * (D + 2) + D + 1] = den;
            }
        } else if (row < valid_rows) {
            const int head = first_head + row;
            if (sink) {
                const float sk = sink[head] * LOG2E, top = fmaxf(big, sk);
                const float f = big == -INFINITY ? 0.0f : exp2f(big - top);
                num *= f;
                den = den * f + exp2f(sk - top);
            }
            float v = den > 0.0f ? num / den : 0.0f;
            if (out_gate) v *= out_gate[(size_t)t * n_heads + head];
            out[(size_t)t * ld_out + (size_t)head * D + col] = __float2bfloat16_rn(v);
        }
    }
}

// Adds the splits' partial rows in the splits' order and finishes the rows.  One thread an element: a thread's loads of
// the splits' values do not depend on one another, so they are in flight together (with a few elements a thread the
// kernel was one long chain of trips to L2: 30 us for 16 splits).
template <int D>
__global__ void __launch_bounds__(128)
decode_shared_merge_kernel(const float* __restrict__ scratch, int splits, bf16* __restrict__ out, int ld_out, int n_heads,
                           int n_kv_heads, const float* __restrict__ sink, const float* __restrict__ out_gate) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.y;
    const int group_heads = n_heads / n_kv_heads, row_tiles = (group_heads + ROWS - 1) / ROWS;
    const int kvh = blockIdx.x / row_tiles, row_tile = blockIdx.x % row_tiles;
    const int first_head = kvh * group_heads + row_tile * ROWS;
    const int valid_rows = min(ROWS, group_heads - row_tile * ROWS);
    const float* base = scratch + ((size_t)t * gridDim.x + blockIdx.x) * splits * ROWS * (D + 2);
    const int idx = blockIdx.z * blockDim.x + threadIdx.x;
    const int row = idx / D, col = idx % D;
    if (row >= valid_rows) return;
    float big = -INFINITY;
#pragma unroll 8
    for (int s = 0; s < splits; s++) big = fmaxf(big, base[((size_t)s * ROWS + row) * (D + 2) + D]);
    float num = 0.0f, den = 0.0f;
#pragma unroll 8
    for (int s = 0; s < splits; s++) {
        const float* p = base + ((size_t)s * ROWS + row) * (D + 2);
        const float f = p[D] == -INFINITY ? 0.0f : exp2f(p[D] - big);
        num = fmaf(f, p[col], num);
        den = fmaf(f, p[D + 1], den);
    }
    const int head = first_head + row;
    if (sink) {
        const float sk = sink[head] * LOG2E, top = fmaxf(big, sk);
        const float f = big == -INFINITY ? 0.0f : exp2f(big - top);
        num *= f;
        den = den * f + exp2f(sk - top);
    }
    float v = den > 0.0f ? num / den : 0.0f;
    if (out_gate) v *= out_gate[(size_t)t * n_heads + head];
    out[(size_t)t * ld_out + (size_t)head * D + col] = __float2bfloat16_rn(v);
}

template <int D>
size_t smem_bytes(bool one_plane) {
    const size_t stages = (size_t)WARPS * STAGES * (one_plane ? 1 : 2) * GROUP * (D + 8) * sizeof(bf16);
    const size_t meet = (size_t)WARPS * ROWS * (D + 2) * sizeof(float);
    return stages > meet ? stages : meet;
}

template <int D>
int launch(const bf16* q, int ld_q, const bf16* k, const bf16* v, long long page_stride, const int* block_table, int max_blocks,
           const int* token_seq, const int* positions, bf16* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int page_size,
           float scale, int window, float softcap, int chunk, int splits, int num_pages, const float* sink, const float* out_gate,
           const float* dist_bias, int n_dist, float* scratch, int* status, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = smem_bytes<D>(k == v);
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(decode_shared_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<D>(false));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group_heads = n_heads / n_kv_heads, tiles = n_kv_heads * ((group_heads + ROWS - 1) / ROWS);
    int code = sandy_launch(decode_shared_kernel<D>, dim3(splits, tiles, n_tokens), dim3(WARPS * 32), smem, stream, q, ld_q, k, v,
                            page_stride, block_table, max_blocks, token_seq, positions, out, ld_out, n_heads, n_kv_heads, page_size,
                            scale, window, softcap, chunk, splits, num_pages, sink, out_gate, dist_bias, n_dist,
                            splits > 1 ? scratch : (float*)nullptr, status);
    if (code != SANDY_OK || splits == 1) return code;
    return sandy_launch(decode_shared_merge_kernel<D>, dim3(tiles, n_tokens, (ROWS * D + 127) / 128), dim3(128), 0, stream, (const float*)scratch, splits, out,
                        ld_out, n_heads, n_kv_heads, sink, out_gate);
}

}  // namespace

// Floats of scratch a launch with more than one split needs.
SANDY_API long long sandy_decode_attention_shared_scratch(int n_tokens, int n_heads, int n_kv_heads, int head_dim, int splits) {
    if (n_kv_heads <= 0 || splits <= 1) return 0;
    const int group_heads = n_heads / n_kv_heads;
    return (long long)n_tokens * n_kv_heads * ((group_heads + ROWS - 1) / ROWS) * splits * ROWS * (head_dim + 2);
}

// q, out: bfloat16 [n_tokens, n_heads * head_dim]; caches bfloat16 [num_pages][n_kv_heads][page_size][head_dim] with
// page_stride elements between pages (v_cache may be k_cache: one plane); one token per request position (a decode
// step).  sink: float32 [n_heads] or null; out_gate: float32 [n_tokens, n_heads] or null.  scratch: float32, as many
// floats as sandy_decode_attention_shared_scratch says (may be null with one split).  softcap > 0: a score becomes
// softcap * tanh(score / softcap); chunk > 0: a query sees only keys j >= pos - pos % chunk.
// dist_bias: float32 [n_heads, n_dist] or null: entry min(pos - j, n_dist - 1) of the head's row joins the score of key j.
SANDY_API int sandy_decode_attention_shared_bias(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                            const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                            void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                            int page_size, float scale, int window, float softcap, int chunk, int splits,
                                            int num_pages, const float* sink, const float* out_gate, const float* dist_bias,
                                            int n_dist, float* scratch, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (dist_bias && n_dist < 1) return SANDY_ERR_ARGUMENT;
    if (!q || !k_cache || !v_cache || !block_table || !token_seq || !positions || !out) return SANDY_ERR_ARGUMENT;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || window < 0 || splits < 1 || splits > 65535 ||
        n_tokens > 65535 || (splits > 1 && !scratch) || softcap < 0.0f || chunk < 0)
        return SANDY_ERR_UNSUPPORTED;
    if (head_dim % 16 || head_dim < 16 || head_dim > 128 || (ld_q & 1) || (page_stride & 7) ||
        ((uintptr_t)q & 3) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return SANDY_ERR_UNSUPPORTED;
#define SANDY_CASE(DD)                                                                                                              \
    case DD:                                                                                                                        \
        return launch<DD>((const bf16*)q, ld_q, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, block_table, max_blocks,  \
                          token_seq, positions, (bf16*)out, ld_out, n_tokens, n_heads, n_kv_heads, page_size, scale, window, softcap, \
                          chunk, splits, num_pages, sink, out_gate, dist_bias, n_dist, scratch, status, stream)
    switch (head_dim) {
        SANDY_CASE(16); SANDY_CASE(32); SANDY_CASE(48); SANDY_CASE(64); SANDY_CASE(80); SANDY_CASE(96); SANDY_CASE(112); SANDY_CASE(128);
    }
#undef SANDY_CASE
    return SANDY_ERR_UNSUPPORTED;
}

// The same without a bias by distance.
SANDY_API int sandy_decode_attention_shared_cap(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                            const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                            void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                            int page_size, float scale, int window, float softcap, int chunk, int splits,
                                            int num_pages, const float* sink, const float* out_gate, float* scratch, int* status,
                                            cudaStream_t stream) {
    return sandy_decode_attention_shared_bias(q, ld_q, k_cache, v_cache, page_stride, block_table, max_blocks, token_seq, positions, out,
                                              ld_out, n_tokens, n_heads, n_kv_heads, head_dim, page_size, scale, window, softcap, chunk,
                                              splits, num_pages, sink, out_gate, nullptr, 0, scratch, status, stream);
}

// The same with plain scores and no chunks.
SANDY_API int sandy_decode_attention_shared(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                            const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                            void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                            int page_size, float scale, int window, int splits, int num_pages, const float* sink,
                                            const float* out_gate, float* scratch, int* status, cudaStream_t stream) {
    return sandy_decode_attention_shared_cap(q, ld_q, k_cache, v_cache, page_stride, block_table, max_blocks, token_seq, positions, out,
                                             ld_out, n_tokens, n_heads, n_kv_heads, head_dim, page_size, scale, window, 0.0f, 0, splits,
                                             num_pages, sink, out_gate, scratch, status, stream);
}
