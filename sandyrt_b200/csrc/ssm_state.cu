// A selective state-space mixer with one decay per head (the recurrence of Mamba-2):
//
//   S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T          S: [N, P] per head, float32, carried from step to step
//   y_t = S_t^T C_t + D x_t                                        heads share B and C in groups
//
//   sandy_ssm_prepare      per token: the short causal convolution (with bias) and silu of the x, B and C channels, rows
//                          before the step's first token of a request from the tail in its state; dt = softplus(raw +
//                          dt_bias) and the decay's logarithm -exp(A_log) dt.  All float32.
//   sandy_ssm_scan         the recurrence, token by token, each request from its own state.  A block owns 4 to 32 columns
//                          of one head's state for one request; 4 to 32 neighbouring threads share a column, each with
//                          every 4th to 32nd group of four rows, so the state update needs no exchange at all and the
//                          read-out y one sum over those neighbouring lanes.  The tokens' inputs reach shared memory eight at a
//                          time by asynchronous copies, the next eight on their way meanwhile.  A step may bring any mix of portions and single tokens.
//   sandy_gated_group_norm out = (y * silu(z)) / rms * gain over `groups` equal parts of a row, the gate BEFORE the norm
//
// The state of a slot is S [H][P][N] (a column's rows are consecutive floats).  Everything is float32 arithmetic whatever
// the engine's compute type; inputs that come from a projection are read in the projection's type.  The recurrence
// stays on the FMA pipe on purpose: the state and everything that enters it are 32-bit by the designs that use it, and
// in this token-by-token form it costs 3 N P operations a token and head, fewer than the chunked forms that trade
// operations for tensor-core shapes.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;
constexpr int THREADS = 128;                   // of the recurrence: columns x the threads that share a column
constexpr int CHUNK = 8;                       // tokens staged at a time

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(256)
ssm_prepare_kernel(const T* __restrict__ proj, int ld, int channels, const float* __restrict__ taps, int n_taps,
                   const float* __restrict__ conv_bias, const float* __restrict__ dt_raw, int ld_dt,
                   const float* __restrict__ dt_bias, const float* __restrict__ a_log, int n_heads,
                   float* __restrict__ state, long long state_stride, long long tail_off,
                   const int* __restrict__ token_seq, const int* __restrict__ q_start, const int* __restrict__ seq_slots,
                   float* __restrict__ xbc, int ld_xbc, float* __restrict__ dta, int keep) {
    const int t = blockIdx.x;
    const int s = token_seq[t];
    const int i_in_step = t - q_start[s];
    float* tail = state + (long long)seq_slots[s] * state_stride + tail_off;      // [n_taps - 1][channels]
    pdl_wait();
    pdl_launch_dependents();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = conv_bias ? conv_bias[c] : 0.0f;
        for (int j = 0; j < n_taps; j++) {
            const int lag = n_taps - 1 - j;
            const int src = i_in_step - lag;
            const float x = src >= 0 ? to_f32(proj[(size_t)(t - lag) * ld + c]) : tail[(size_t)(n_taps - 1 + src) * channels + c];
            y = fmaf(taps[(size_t)c * n_taps + j], x, y);
        }
        xbc[(size_t)t * ld_xbc + c] = silu_f(y);
        // a step of single tokens: the tail moves on by this token here (this thread alone reads and writes its channel)
        if (keep && n_taps > 1) {
            for (int j = 0; j + 2 < n_taps; j++) tail[(size_t)j * channels + c] = tail[(size_t)(j + 1) * channels + c];
            tail[(size_t)(n_taps - 2) * channels + c] = to_f32(proj[(size_t)t * ld + c]);
        }
    }
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        const float dt = softplus_f(dt_raw[(size_t)t * ld_dt + h] + dt_bias[h]);
        dta[(size_t)t * 2 * n_heads + h] = dt;
        dta[(size_t)t * 2 * n_heads + n_heads + h] = -expf(a_log[h]) * dt;
    }
}

// xbc: float32 [T, ld] rows of (x [H * P], B [G * N], C [G * N]); dta: float32 [T, 2H] (dt, then the decay's logarithm).
// SL: threads that share a column (each owns every SL-th group of four rows); Q: groups of four rows a thread owns; rows
// beyond N are zeros.  What a token brings to a block, as it lies in shared memory: B [4 Q SL], C [4 Q SL], x [COLS], dt,
// the decay's logarithm.
template <int Q, int SL>
__global__ void __launch_bounds__(THREADS)
ssm_scan_kernel(const float* __restrict__ xbc, int ld, const float* __restrict__ dta, const float* __restrict__ d_skip,
                float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                const int* __restrict__ seq_slots, float* __restrict__ out, int ld_out, int n_heads, int n_groups, int N, int P,
                int wide) {
    constexpr int NP = 4 * Q * SL;
    constexpr int COLS = THREADS / SL;               // columns of a head's state per block
    constexpr int PER = 2 * NP + COLS + 4;           // dt, the decay's logarithm, and two floats that keep a token's rows 16-byte aligned
    static_assert(COLS % 4 == 0, "a token's rows stay 16-byte aligned");
    __shared__ __align__(16) float stage[2][CHUNK * PER];
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
    const int slice = threadIdx.x % SL, col = col0 + threadIdx.x / SL;
    const int g = h / (n_heads / n_groups);
    const int t0 = q_start[s], t1 = q_start[s + 1];
    const int inner = n_heads * P;
    const float skip = d_skip ? d_skip[h] : 0.0f;
    float* S = state + (long long)seq_slots[s] * state_stride + ((long long)h * P + col) * N;
    // What this thread copies for every token: elements tid, tid + THREADS, ... of the token's PER floats.  Where each
    // comes from is the same for every token, so it is worked out once: an offset into the token's row of xbc, or one of
    // the two gate numbers, or nothing (zeros: rows beyond N, columns beyond P, padding).
    constexpr int NY = (PER + THREADS - 1) / THREADS;
    int src[NY];
#pragma unroll
    for (int y = 0; y < NY; y++) {
        const int e = threadIdx.x + y * THREADS;
        int o = -1;
        if (e < NP) o = e < N ? inner + g * N + e : -1;
        else if (e < 2 * NP) o = e - NP < N ? inner + n_groups * N + g * N + (e - NP) : -1;
        else if (e < 2 * NP + COLS) o = col0 + e - 2 * NP < P ? h * P + col0 + e - 2 * NP : -1;
        else if (e == 2 * NP + COLS) o = -2;
        else if (e == 2 * NP + COLS + 1) o = -3;
        src[y] = o;
    }
    pdl_wait();
    float st[Q][4];
#pragma unroll
    for (int q = 0; q < Q; q++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int n = 4 * (q * SL + slice) + e;
            st[q][e] = (col < P && n < N) ? S[n] : 0.0f;
        }
    // Eight tokens' inputs go from global to shared memory by asynchronous copies (zeros where there is nothing), into
    // the buffer that is not being read: they are on their way while the eight before are computed.  Where every row
    // starts on a 16-byte boundary (`wide`) B, C and x travel sixteen bytes a copy, else four.
    constexpr int NV = (PER / 4 + THREADS - 1) / THREADS;
    int vsrc[NV];
#pragma unroll
    for (int y = 0; y < NV; y++) {
        const int e = 4 * (threadIdx.x + y * THREADS);       // first float of this thread's piece
        int o = -1;
        if (e < NP) o = e < N ? inner + g * N + e : -1;
        else if (e < 2 * NP) o = e - NP < N ? inner + n_groups * N + g * N + (e - NP) : -1;
        else if (e < 2 * NP + COLS) o = col0 + e - 2 * NP < P ? h * P + col0 + e - 2 * NP : -1;
        else if (e == 2 * NP + COLS) o = -2;                 // dt and the decay's logarithm: two copies of four bytes
        vsrc[y] = o;
    }
    auto fetch = [&](int tc, int buf) {
        const int n_tok = min(CHUNK, t1 - tc);
        if (wide) {
#pragma unroll
            for (int tok = 0; tok < CHUNK; tok++) {
                const float* row = xbc + (size_t)(tc + tok) * ld;
#pragma unroll
                for (int y = 0; y < NV; y++) {
                    const int e = 4 * (threadIdx.x + y * THREADS);
                    if (e >= PER) continue;
                    const unsigned dst = (unsigned)__cvta_generic_to_shared(&stage[buf][tok * PER + e]);
                    if (vsrc[y] == -2) {
                        const float* gates = dta + (size_t)(tc + tok) * 2 * n_heads + h;
                        const int bytes = tok < n_tok ? 4 : 0;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(gates), "r"(bytes) : "memory");
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + 4), "l"(gates + n_heads), "r"(bytes) : "memory");
                    } else {
                        const bool real = tok < n_tok && vsrc[y] >= 0;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(real ? row + vsrc[y] : xbc), "r"(real ? 16 : 0) : "memory");
                    }
                }
            }
        } else {
#pragma unroll
            for (int tok = 0; tok < CHUNK; tok++) {
                const float* row = xbc + (size_t)(tc + tok) * ld;
                const float* gates = dta + (size_t)(tc + tok) * 2 * n_heads + h;
#pragma unroll
                for (int y = 0; y < NY; y++) {
                    const int e = threadIdx.x + y * THREADS;
                    if (e < PER) {
                        const bool real = tok < n_tok && src[y] != -1;
                        const float* from = !real ? xbc : src[y] >= 0 ? row + src[y] : src[y] == -2 ? gates : gates + n_heads;
                        const unsigned dst = (unsigned)__cvta_generic_to_shared(&stage[buf][tok * PER + e]);
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(from), "r"(real ? 4 : 0) : "memory");
                    }
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (t0 < t1) fetch(t0, 0);
    int buf = 0;
    for (int tc = t0; tc < t1; tc += CHUNK, buf ^= 1) {
        if (tc + CHUNK < t1) {
            fetch(tc + CHUNK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int n_tok = min(CHUNK, t1 - tc);
        for (int tok = 0; tok < n_tok; tok++) {
            const float* in = stage[buf] + tok * PER;
            const float xv = in[2 * NP + threadIdx.x / SL];
            const float dt = in[2 * NP + COLS], decay = expf(in[2 * NP + COLS + 1]);
            const float dtx = dt * xv;
            float y0 = 0.0f, y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;      // four chains: a token's read-out is not one long chain of additions
#pragma unroll
            for (int q = 0; q < Q; q++) {
                const float4 b = *reinterpret_cast<const float4*>(in + 4 * (q * SL + slice));
                const float4 c = *reinterpret_cast<const float4*>(in + NP + 4 * (q * SL + slice));
                st[q][0] = fmaf(b.x, dtx, decay * st[q][0]);
                st[q][1] = fmaf(b.y, dtx, decay * st[q][1]);
                st[q][2] = fmaf(b.z, dtx, decay * st[q][2]);
                st[q][3] = fmaf(b.w, dtx, decay * st[q][3]);
                y0 = fmaf(st[q][0], c.x, y0);
                y1 = fmaf(st[q][1], c.y, y1);
                y2 = fmaf(st[q][2], c.z, y2);
                y3 = fmaf(st[q][3], c.w, y3);
            }
            float y = (y0 + y1) + (y2 + y3);
#pragma unroll
            for (int o = 1; o < SL; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);      // the SL threads of a column are neighbours
            if (slice == 0 && col < P) out[(size_t)(tc + tok) * ld_out + h * P + col] = fmaf(skip, xv, y);
        }
        __syncthreads();             // everyone is done with this buffer before the copies after next land in it
    }
    pdl_launch_dependents();
    if (t0 < t1 && col < P) {
#pragma unroll
        for (int q = 0; q < Q; q++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int n = 4 * (q * SL + slice) + e;
                if (n < N) S[n] = st[q][e];
            }
    }
}

// One block per (token, part of the row).
template <typename T>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, int ldy, const T* __restrict__ z, int ldz, const float* __restrict__ gain,
                        float eps, int part, T* __restrict__ out, int ld_out) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    pdl_wait();
    pdl_launch_dependents();
    float ss = 0.0f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float v = y[(size_t)t * ldy + c0 + i] * silu_f(to_f32(z[(size_t)t * ldz + c0 + i]));
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float v = y[(size_t)t * ldy + c0 + i] * silu_f(to_f32(z[(size_t)t * ldz + c0 + i]));
        out[(size_t)t * ld_out + c0 + i] = from_f32<T>(v * inv * (gain ? gain[c0 + i] : 1.0f));
    }
}

}  // namespace

SANDY_API long long sandy_ssm_state_floats(int n_heads, int state, int v_dim) { return (long long)n_heads * state * v_dim; }

// proj: [n_tokens, >= channels] of dtype with pitch ld, the x, B and C channels first (the caller passes the address of
// their first column).  taps float32 [channels, n_taps], conv_bias float32 [channels] or null.  dt_raw float32
// [n_tokens, >= n_heads] with pitch ld_dt.  The tail of a slot is float32 [n_taps - 1][channels] at tail_off of its state.
// xbc float32 [n_tokens, channels] with pitch ld_xbc; dta float32 [n_tokens, 2 * n_heads].  keep != 0 (only right when every
// request brings one token): the tails move on by the step's tokens in this launch; otherwise sandy_conv_tail follows.
SANDY_API int sandy_ssm_prepare(const void* proj, int ld, int dtype, int channels, const float* taps, int n_taps,
                                const float* conv_bias, const float* dt_raw, int ld_dt, const float* dt_bias, const float* a_log,
                                int n_heads, float* state, long long state_stride, long long tail_off,
                                const int* token_seq, const int* q_start, const int* seq_slots, float* xbc, int ld_xbc,
                                float* dta, int n_tokens, int keep, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!proj || !taps || !dt_raw || !dt_bias || !a_log || !token_seq || !q_start || !seq_slots || !xbc || !dta ||
        (n_taps > 1 && !state))
        return SANDY_ERR_ARGUMENT;
    if (n_taps < 1 || n_taps > MAX_TAPS || channels < 1 || n_heads < 1) return SANDY_ERR_UNSUPPORTED;
    if (dtype == SANDY_F32)
        return sandy_launch(ssm_prepare_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)proj, ld, channels, taps,
                            n_taps, conv_bias, dt_raw, ld_dt, dt_bias, a_log, n_heads, state, state_stride, tail_off, token_seq,
                            q_start, seq_slots, xbc, ld_xbc, dta, keep);
    if (dtype == SANDY_BF16)
        return sandy_launch(ssm_prepare_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, (const bf16*)proj, ld, channels, taps,
                            n_taps, conv_bias, dt_raw, ld_dt, dt_bias, a_log, n_heads, state, state_stride, tail_off, token_seq,
                            q_start, seq_slots, xbc, ld_xbc, dta, keep);
    return SANDY_ERR_UNSUPPORTED;
}

// d_skip float32 [n_heads] or null; out float32 [n_tokens, n_heads * v_dim].  state (N) up to 256.
SANDY_API int sandy_ssm_scan(const float* xbc, int ld, const float* dta, const float* d_skip, float* state, long long state_stride,
                             const int* q_start, const int* seq_slots, float* out, int ld_out, int n_seqs, int n_heads,
                             int n_groups, int state_dim, int v_dim, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!xbc || !dta || !state || !q_start || !seq_slots || !out) return SANDY_ERR_ARGUMENT;
    if (n_heads < 1 || n_groups < 1 || n_heads % n_groups || state_dim < 1 || state_dim > 256 || v_dim < 1)
        return SANDY_ERR_UNSUPPORTED;
#define SCAN(Q, SL)                                                                                                          \
    do {                                                                                                                     \
        const dim3 grid(n_seqs, n_heads, (v_dim + THREADS / SL - 1) / (THREADS / SL));                                       \
        if (grid.y > 65535 || grid.z > 65535) return SANDY_ERR_UNSUPPORTED;                                                  \
        return sandy_launch(ssm_scan_kernel<Q, SL>, grid, dim3(THREADS), 0, stream, xbc, ld, dta, d_skip, state, state_stride, \
                            q_start, seq_slots, out, ld_out, n_heads, n_groups, state_dim, v_dim, wide);                     \
    } while (0)
    // rows of B, C and x that all start on 16-byte boundaries travel sixteen bytes a copy
    const int wide = state_dim % 4 == 0 && v_dim % 4 == 0 && ld % 4 == 0 && ((uintptr_t)xbc & 15) == 0 ? 1 : 0;
    // a thread owns four rows of its column (eight from a state of 129 on): the tokens of a request come one after
    // another, so what a token costs is the length of a thread's chain of instructions, and the more threads share a
    // column the shorter it is and the more warps an SM has to choose from
    if (state_dim <= 16) SCAN(1, 4);
    if (state_dim <= 32) SCAN(1, 8);
    if (state_dim <= 64) SCAN(1, 16);
    if (state_dim <= 128) SCAN(1, 32);
    SCAN(2, 32);
#undef SCAN
}

// y float32 [n_tokens, cols]; z and out [n_tokens, cols] of dtype; gain float32 [cols] or null; cols = groups * part.
SANDY_API int sandy_gated_group_norm(const float* y, int ldy, const void* z, int ldz, const float* gain, float eps, int groups,
                                     void* out, int ld_out, int n_tokens, int cols, int dtype, cudaStream_t stream) {
    if (n_tokens == 0 || cols == 0) return SANDY_OK;
    if (!y || !z || !out) return SANDY_ERR_ARGUMENT;
    if (groups < 1 || cols % groups || groups > 65535) return SANDY_ERR_UNSUPPORTED;
    const int part = cols / groups;
    if (dtype == SANDY_F32)
        return sandy_launch(gated_group_norm_kernel<float>, dim3(n_tokens, groups), dim3(256), 0, stream, y, ldy, (const float*)z, ldz,
                            gain, eps, part, (float*)out, ld_out);
    if (dtype == SANDY_BF16)
        return sandy_launch(gated_group_norm_kernel<bf16>, dim3(n_tokens, groups), dim3(256), 0, stream, y, ldy, (const bf16*)z, ldz,
                            gain, eps, part, (bf16*)out, ld_out);
    return SANDY_ERR_UNSUPPORTED;
}
