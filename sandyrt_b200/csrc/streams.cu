// A residual stream kept in several copies (hyper-connections), and what surrounds a sublayer that reads it.
//
// The stream of a token is S rows of `width` floats, X[t] = [X_1 | X_2 | ... | X_S], all float32.  A sublayer reads
// one mixture of them and writes into all of them:
//
//   u      = sum_s in[s] X_s                                    what the sublayer's norm sees
//   h      = (u - mean) / sqrt(var + eps) * gain                LayerNorm without an offset (biased variance, two passes)
//   y      = sublayer(...)                                       somewhere else
//   X_t   <- sum_s mix[s, t] X_s + out[t] * y * sigmoid(g + b)   g: the pre-activations of a gate on the sublayer's result
//
//   sandy_streams_step     for every token, in this order and each part optional: the write of one sublayer's result
//                          into the streams, the read (and norm) for the next sublayer, and the plain sum of the streams
//                          (what the model's final norm reads).  One block a token; a token's S rows stay in registers
//                          between the parts, so a write followed by a read costs one pass over the streams.  In a step of
//                          single tokens the same launch also runs the short convolution below and moves its tail on.
//   sandy_streams_spread   X_s = x for every s: the embedding's output enters all streams
//   sandy_canon_conv       c[t] = h[t] + sum_k taps[:, k] h[t - n + 1 + k]: a short causal convolution over time on every
//                          channel, added to its own input; rows before the step's first token of a request come from
//                          the tail kept in the request's state (zeros at a request's start)
//   sandy_embed_bigram     x[t] = E[id_t] + B[(id_{t-1} a + id_t b) mod n] + P[pos_t]; a request's first token reads row n
//                          of B; the token before a step's first one is kept in the request's state
//   sandy_bigram_keep      the state takes each request's last token of the step
//
// Everything is computed in float32; h and c are rounded once, to the compute type, when they are written.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int BIG = 1024;                       // threads of a block when a step has few tokens
constexpr int MAX_STREAMS = 8;
constexpr int MAX_PER_THREAD = 8;              // channels a thread keeps in registers: widths up to 2,048
constexpr int MAX_TAPS = 8;

// One token's row on TH threads.  PER > 0: width <= PER * TH and the streams stay in registers; PER == 0: any width, the
// streams are read again where they are needed (they were written by this thread, so no barrier lies between).
template <typename T, int S_MAX, int PER, int TH>
__global__ void __launch_bounds__(TH)
streams_step_kernel(float* __restrict__ X, int ldX, int n_streams, int width,
                    const float* __restrict__ y, int ldy, const float* __restrict__ gate, int ldg,
                    const float* __restrict__ gate_bias, const float* __restrict__ mix, const float* __restrict__ out_w,
                    const float* __restrict__ in_w, const float* __restrict__ gain, float eps, T* __restrict__ h, int ldh,
                    float* __restrict__ sum_out, int ld_sum, const float* __restrict__ taps, int n_taps, float* __restrict__ state,
                    long long state_stride, long long tail_off, const int* __restrict__ token_seq,
                    const int* __restrict__ seq_slots, T* __restrict__ c, int ldc) {
    __shared__ float scratch[32];
    __shared__ float coef[S_MAX * S_MAX + 2 * S_MAX];
    const int t = blockIdx.x;
    const int S = n_streams;
    // the small tables are weights: they may be read before the kernel in front has ended
    for (int i = threadIdx.x; i < S * S + 2 * S; i += TH) {
        float v = 0.0f;
        if (i < S * S) v = mix ? mix[i] : 0.0f;
        else if (i < S * S + S) v = out_w ? out_w[i - S * S] : 0.0f;
        else v = in_w ? in_w[i - S * S - S] : 0.0f;
        coef[i] = v;
    }
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    float* row = X + (size_t)t * ldX;
    constexpr int P = PER > 0 ? PER : 1;
    float u[P];
    float total = 0.0f;
    const int rounds = PER > 0 ? PER : (width + TH - 1) / TH;
    for (int r = 0; r < rounds; r++) {
        const int j = threadIdx.x + r * TH;
        float uj = 0.0f;
        if (j < width) {
            float x[S_MAX];
#pragma unroll
            for (int s = 0; s < S_MAX; s++) x[s] = s < S ? row[(size_t)s * width + j] : 0.0f;
            if (y) {
                const float z = gate[(size_t)t * ldg + j] + gate_bias[j];
                const float branch = y[(size_t)t * ldy + j] / (1.0f + expf(-z));
                float nx[S_MAX];
#pragma unroll
                for (int to = 0; to < S_MAX; to++) {
                    float a = 0.0f;
                    if (to < S) {
#pragma unroll
                        for (int s = 0; s < S_MAX; s++)
                            if (s < S) a = fmaf(coef[s * S + to], x[s], a);
                        a = fmaf(coef[S * S + to], branch, a);
                    }
                    nx[to] = a;
                }
#pragma unroll
                for (int s = 0; s < S_MAX; s++) {
                    x[s] = nx[s];
                    if (s < S) row[(size_t)s * width + j] = x[s];
                }
            }
            if (sum_out) {
                float a = 0.0f;
#pragma unroll
                for (int s = 0; s < S_MAX; s++)
                    if (s < S) a += x[s];
                sum_out[(size_t)t * ld_sum + j] = a;
            }
            if (in_w) {
#pragma unroll
                for (int s = 0; s < S_MAX; s++)
                    if (s < S) uj = fmaf(coef[S * S + S + s], x[s], uj);
            }
        }
        if (PER > 0) u[r] = uj;
        total += uj;
    }
    if (!in_w) return;
    auto u_at = [&](int r, int j) -> float {
        if (PER > 0) return u[r];
        float a = 0.0f;
        for (int s = 0; s < S; s++) a = fmaf(coef[S * S + S + s], row[(size_t)s * width + j], a);
        return a;
    };
    const float mean = block_sum(total, scratch) / (float)width;
    float sq = 0.0f;
    for (int r = 0; r < rounds; r++) {
        const int j = threadIdx.x + r * TH;
        if (j < width) {
            const float d = u_at(r, j) - mean;
            sq = fmaf(d, d, sq);
        }
    }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    // A step of single tokens runs the short convolution here too: c = h + conv(h) from the request's tail, which then
    // moves on by this token (a thread owns its channels of the tail: nobody else reads or writes them in this step).
    float* tail = taps && n_taps > 1 ? state + (long long)seq_slots[token_seq[t]] * state_stride + tail_off : nullptr;
    for (int r = 0; r < rounds; r++) {
        const int j = threadIdx.x + r * TH;
        if (j < width) {
            const T rounded = from_f32<T>((u_at(r, j) - mean) * rstd * gain[j]);
            h[(size_t)t * ldh + j] = rounded;
            if (taps) {
                const float own = to_f32(rounded);
                float a = taps[(size_t)j * n_taps + n_taps - 1] * own;
                for (int k = 0; k + 1 < n_taps; k++) {
                    const float x = tail[(size_t)k * width + j];
                    a = fmaf(taps[(size_t)j * n_taps + k], x, a);
                    if (k > 0) tail[(size_t)(k - 1) * width + j] = x;
                }
                if (n_taps > 1) tail[(size_t)(n_taps - 2) * width + j] = own;
                c[(size_t)t * ldc + j] = from_f32<T>(own + a);
            }
        }
    }
}

__global__ void __launch_bounds__(THREADS)
streams_spread_kernel(const float* __restrict__ x, int ldx, float* __restrict__ X, int ldX, int n_tokens, int n_streams, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long)n_tokens * n_streams * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / ((long long)n_streams * width), r = i % ((long long)n_streams * width);
        X[t * ldX + r] = x[t * ldx + r % width];
    }
}

// h, c: [T, width] of T.  taps float32 [width, n_taps], the last column the token's own.  tail: the request's last
// n_taps - 1 rows of h before the step, float32 [n_taps - 1][width] at tail_off of its state row.
template <typename T>
__global__ void __launch_bounds__(THREADS)
canon_conv_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ taps, int n_taps, const float* __restrict__ state,
                  long long state_stride, long long tail_off, const int* __restrict__ token_seq, const int* __restrict__ q_start,
                  const int* __restrict__ seq_slots, T* __restrict__ c, int ldc, int n_tokens, int width) {
    const int t = blockIdx.x;                        // a block a token
    const int s = token_seq[t];
    const int i_in_step = t - q_start[s];
    const float* tail = state + (long long)seq_slots[s] * state_stride + tail_off;
    pdl_wait();
    pdl_launch_dependents();
    for (int j = threadIdx.x; j < width; j += THREADS) {
        const float own = to_f32(h[(size_t)t * ldh + j]);
        float a = 0.0f;
        for (int k = 0; k < n_taps; k++) {
            const int lag = n_taps - 1 - k;
            const int src = i_in_step - lag;
            const float x = lag == 0 ? own : (src >= 0 ? to_f32(h[(size_t)(t - lag) * ldh + j]) : tail[(size_t)(n_taps - 1 + src) * width + j]);
            a = fmaf(taps[(size_t)j * n_taps + k], x, a);
        }
        c[(size_t)t * ldc + j] = from_f32<T>(own + a);
    }
    (void)n_tokens;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
embed_bigram_kernel(const int* __restrict__ ids, const int* __restrict__ positions, const int* __restrict__ token_seq,
                    const int* __restrict__ q_start, const int* __restrict__ seq_slots, const T* __restrict__ wte,
                    const T* __restrict__ bigram, const T* __restrict__ wpe, int buckets, long long mul_prev, long long mul_cur,
                    int* __restrict__ state, long long state_stride, float* __restrict__ x, int ldx, int vocab, int n_pos,
                    int width, int keep, int* __restrict__ status) {
    const int t = blockIdx.x;
    pdl_wait();                              // the first kernel of a step: nothing of the step may start before the steps before have ended
    pdl_launch_dependents();
    const int id = ids[t], pos = positions[t];
    const int s = token_seq[t];
    const int first = q_start[s];
    int* slot = state + (long long)seq_slots[s] * state_stride;
    const bool bad_id = id < 0 || id >= vocab, bad_pos = pos < 0 || (wpe && pos >= n_pos);
    int prev = 0;
    if (pos > 0) prev = t > first ? ids[t - 1] : slot[0];
    if (prev < 0 || prev >= vocab) prev = 0;              // reported through its own token's id
    if (bad_id || bad_pos) {
        if (threadIdx.x == 0 && status) atomicOr(status, bad_id ? 1 : 2);
        for (int j = threadIdx.x; j < width; j += THREADS) x[(size_t)t * ldx + j] = 0.0f;
        return;
    }
    // ids and multipliers are below 2^31 each: the sum of the two products stays below 2^63, which unsigned 64-bit arithmetic holds
    const long long brow = pos == 0 ? (long long)buckets
                                    : (long long)(((unsigned long long)prev * (unsigned long long)mul_prev +
                                                   (unsigned long long)id * (unsigned long long)mul_cur) % (unsigned long long)buckets);
    const T* e = wte + (size_t)id * width;
    const T* b = bigram + (size_t)brow * width;
    const T* p = wpe ? wpe + (size_t)pos * width : nullptr;
    for (int j = threadIdx.x; j < width; j += THREADS)
        x[(size_t)t * ldx + j] = to_f32(e[j]) + to_f32(b[j]) + (p ? to_f32(p[j]) : 0.0f);
    // a step of single tokens keeps the token here: this block is the only one that reads or writes the slot
    if (keep && threadIdx.x == 0) slot[0] = id;
}

__global__ void bigram_keep_kernel(const int* __restrict__ ids, const int* __restrict__ q_start, const int* __restrict__ seq_slots,
                                   int* __restrict__ state, long long state_stride, int n_seqs) {
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_seqs) return;
    const int t1 = q_start[s + 1];
    if (t1 > q_start[s]) state[(long long)seq_slots[s] * state_stride] = ids[t1 - 1];
}

inline unsigned blocks_for(long long n) {
    const long long want = (n + THREADS - 1) / THREADS;
    const long long cap = (long long)sandy_sm_count() * 16;
    return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

template <typename T>
int launch_step(float* X, int ldX, int n_tokens, int S, int width, const float* y, int ldy, const float* gate, int ldg,
                const float* gate_bias, const float* mix, const float* out_w, const float* in_w, const float* gain, float eps,
                T* h, int ldh, float* sum_out, int ld_sum, const float* taps, int n_taps, float* state, long long state_stride,
                long long tail_off, const int* token_seq, const int* seq_slots, T* c, int ldc, cudaStream_t stream) {
#define STEP(SM, PER, TH)                                                                                                    \
    return sandy_launch(streams_step_kernel<T, SM, PER, TH>, dim3(n_tokens), dim3(TH), 0, stream, X, ldX, S, width, y, ldy,  \
                        gate, ldg, gate_bias, mix, out_w, in_w, gain, eps, h, ldh, sum_out, ld_sum, taps, n_taps, state,      \
                        state_stride, tail_off, token_seq, seq_slots, c, ldc)
    // A step of few tokens (a decode step) leaves most SMs without a block: a token's row then goes over 1,024 threads, a
    // channel or two each, so that the chain of loads and the two sums a thread walks is short.  Many tokens: 256 threads.
    const bool few = n_tokens < sandy_sm_count() && width > THREADS;
    if (S <= 2) {
        if (few && width <= BIG) STEP(2, 1, BIG);
        if (few && width <= 2 * BIG) STEP(2, 2, BIG);
        if (width <= 2 * THREADS) STEP(2, 2, THREADS);
        if (width <= 4 * THREADS) STEP(2, 4, THREADS);
        if (width <= MAX_PER_THREAD * THREADS) STEP(2, MAX_PER_THREAD, THREADS);
        STEP(2, 0, THREADS);
    }
    if (S <= 4) {
        if (few && width <= BIG) STEP(4, 1, BIG);
        if (few && width <= 2 * BIG) STEP(4, 2, BIG);
        if (width <= 4 * THREADS) STEP(4, 4, THREADS);
        if (width <= MAX_PER_THREAD * THREADS) STEP(4, MAX_PER_THREAD, THREADS);
        STEP(4, 0, THREADS);
    }
    if (few && width <= BIG) STEP(MAX_STREAMS, 1, BIG);
    if (width <= 4 * THREADS) STEP(MAX_STREAMS, 4, THREADS);
    STEP(MAX_STREAMS, 0, THREADS);
#undef STEP
}

}  // namespace

// X: float32 [n_tokens, n_streams * width] with pitch ldX, updated in place.
// Write (y != null): y float32 [n_tokens, width], gate float32 [n_tokens, width] and gate_bias float32 [width] (the branch
//   is y * sigmoid(gate + gate_bias)), mix float32 [n_streams, n_streams] indexed [from, to], out_w float32 [n_streams].
// Read (in_w != null): in_w float32 [n_streams], gain float32 [width], eps; h [n_tokens, width] of h_dtype.
// Sum (sum_out != null): float32 [n_tokens, width] = the sum of the streams (after the write).
// Convolution (taps != null, only with the read and ONLY in a step in which every request brings one token): c = h + conv(h)
//   as sandy_canon_conv gives it, [n_tokens, width] of h_dtype, and the request's tail (float32 [n_taps - 1][width] at tail_off
//   of its row of `state`) moved on by the token.
SANDY_API int sandy_streams_step_conv(float* X, int ldX, int n_tokens, int n_streams, int width, const float* y, int ldy,
                                      const float* gate, int ldg, const float* gate_bias, const float* mix, const float* out_w,
                                      const float* in_w, const float* gain, float eps, void* h, int ldh, int h_dtype,
                                      float* sum_out, int ld_sum, const float* taps, int n_taps, float* state,
                                      long long state_stride, long long tail_off, const int* token_seq, const int* seq_slots,
                                      void* c, int ldc, cudaStream_t stream) {
    if (n_tokens == 0 || width == 0) return SANDY_OK;
    if (!X || (y && (!gate || !gate_bias || !mix || !out_w)) || (in_w && (!gain || !h))) return SANDY_ERR_ARGUMENT;
    if (taps && (!in_w || !c || n_taps < 1 || n_taps > MAX_TAPS || (n_taps > 1 && (!state || !token_seq || !seq_slots)))) return SANDY_ERR_ARGUMENT;
    if (n_streams < 1 || n_streams > MAX_STREAMS) return SANDY_ERR_UNSUPPORTED;
    if (h_dtype == SANDY_F32)
        return launch_step<float>(X, ldX, n_tokens, n_streams, width, y, ldy, gate, ldg, gate_bias, mix, out_w, in_w, gain, eps,
                                  (float*)h, ldh, sum_out, ld_sum, taps, n_taps, state, state_stride, tail_off, token_seq, seq_slots,
                                  (float*)c, ldc, stream);
    if (h_dtype == SANDY_BF16)
        return launch_step<bf16>(X, ldX, n_tokens, n_streams, width, y, ldy, gate, ldg, gate_bias, mix, out_w, in_w, gain, eps,
                                 (bf16*)h, ldh, sum_out, ld_sum, taps, n_taps, state, state_stride, tail_off, token_seq, seq_slots,
                                 (bf16*)c, ldc, stream);
    return SANDY_ERR_UNSUPPORTED;
}

// The same without the convolution.
SANDY_API int sandy_streams_step(float* X, int ldX, int n_tokens, int n_streams, int width, const float* y, int ldy,
                                 const float* gate, int ldg, const float* gate_bias, const float* mix, const float* out_w,
                                 const float* in_w, const float* gain, float eps, void* h, int ldh, int h_dtype, float* sum_out,
                                 int ld_sum, cudaStream_t stream) {
    return sandy_streams_step_conv(X, ldX, n_tokens, n_streams, width, y, ldy, gate, ldg, gate_bias, mix, out_w, in_w, gain, eps, h, ldh,
                                   h_dtype, sum_out, ld_sum, nullptr, 0, nullptr, 0, 0, nullptr, nullptr, nullptr, 0, stream);
}

SANDY_API int sandy_streams_max(void) { return MAX_STREAMS; }

SANDY_API int sandy_streams_spread(const float* x, int ldx, float* X, int ldX, int n_tokens, int n_streams, int width,
                                   cudaStream_t stream) {
    if (n_tokens == 0 || width == 0) return SANDY_OK;
    if (!x || !X || n_streams < 1) return SANDY_ERR_ARGUMENT;
    return sandy_launch(streams_spread_kernel, dim3(blocks_for((long long)n_tokens * n_streams * width)), dim3(THREADS), 0, stream, x,
                        ldx, X, ldX, n_tokens, n_streams, width);
}

// h and c: [n_tokens, width] of dtype (they may not be the same buffer: a token reads its neighbours' h).
SANDY_API int sandy_canon_conv(const void* h, int ldh, const float* taps, int n_taps, const float* state, long long state_stride,
                               long long tail_off, const int* token_seq, const int* q_start, const int* seq_slots, void* c,
                               int ldc, int n_tokens, int width, int dtype, cudaStream_t stream) {
    if (n_tokens == 0 || width == 0) return SANDY_OK;
    if (!h || !taps || !c || !token_seq || !q_start || !seq_slots || (n_taps > 1 && !state) || h == c) return SANDY_ERR_ARGUMENT;
    if (n_taps < 1 || n_taps > MAX_TAPS) return SANDY_ERR_UNSUPPORTED;
    const unsigned grid = (unsigned)n_tokens;
    if (dtype == SANDY_F32)
        return sandy_launch(canon_conv_kernel<float>, dim3(grid), dim3(THREADS), 0, stream, (const float*)h, ldh, taps, n_taps, state,
                            state_stride, tail_off, token_seq, q_start, seq_slots, (float*)c, ldc, n_tokens, width);
    if (dtype == SANDY_BF16)
        return sandy_launch(canon_conv_kernel<bf16>, dim3(grid), dim3(THREADS), 0, stream, (const bf16*)h, ldh, taps, n_taps, state,
                            state_stride, tail_off, token_seq, q_start, seq_slots, (bf16*)c, ldc, n_tokens, width);
    return SANDY_ERR_UNSUPPORTED;
}

// wte [vocab, width], bigram [buckets + 1, width], wpe [n_pos, width] or null, all of table_dtype; x float32 [n_tokens, width].
// state: int32, one number a slot at pitch state_stride (the request's last token).  keep != 0: this launch also keeps the
// tokens (only right when every request brings one token); otherwise sandy_bigram_keep follows.
SANDY_API int sandy_embed_bigram(const int* ids, const int* positions, const int* token_seq, const int* q_start,
                                 const int* seq_slots, const void* wte, const void* bigram, const void* wpe, int buckets,
                                 long long mul_prev, long long mul_cur, int* state, long long state_stride, float* x, int ldx,
                                 int n_tokens, int vocab, int n_pos, int width, int table_dtype, int keep, int* status,
                                 cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!ids || !positions || !token_seq || !q_start || !seq_slots || !wte || !bigram || !state || !x) return SANDY_ERR_ARGUMENT;
    if (buckets < 1 || mul_prev < 0 || mul_cur < 0) return SANDY_ERR_UNSUPPORTED;
    if (table_dtype == SANDY_F32)
        return sandy_launch(embed_bigram_kernel<float>, dim3(n_tokens), dim3(THREADS), 0, stream, ids, positions, token_seq, q_start,
                            seq_slots, (const float*)wte, (const float*)bigram, (const float*)wpe, buckets, mul_prev, mul_cur, state,
                            state_stride, x, ldx, vocab, n_pos, width, keep, status);
    if (table_dtype == SANDY_BF16)
        return sandy_launch(embed_bigram_kernel<bf16>, dim3(n_tokens), dim3(THREADS), 0, stream, ids, positions, token_seq, q_start,
                            seq_slots, (const bf16*)wte, (const bf16*)bigram, (const bf16*)wpe, buckets, mul_prev, mul_cur, state,
                            state_stride, x, ldx, vocab, n_pos, width, keep, status);
    return SANDY_ERR_UNSUPPORTED;
}

SANDY_API int sandy_bigram_keep(const int* ids, const int* q_start, const int* seq_slots, int* state, long long state_stride,
                                int n_seqs, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!ids || !q_start || !seq_slots || !state) return SANDY_ERR_ARGUMENT;
    return sandy_launch(bigram_keep_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, ids, q_start, seq_slots, state,
                        state_stride, n_seqs);
}
