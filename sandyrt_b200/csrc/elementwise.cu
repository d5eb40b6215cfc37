// Small element-wise kernels between the products of a layer.
//
//   sandy_glu         out[t, j] = act(a[t, j]) * b[t, j]     a gated feed-forward's inner activation: a and b are the
//                                                            two halves of one fused up-projection
//   sandy_cast_cols   out[t, c0 + j] = x[t, j]               float32 rows rounded into a column range of a wider matrix
//                                                            of the compute type (the operand [x; x0] of a product
//                                                            over two streams side by side)
//   sandy_scale_add   x[t, j] += gain[j] * y[t, j]           a sublayer's result joins the stream through a learned
//                                                            factor per channel (layer scale); all float32
//   sandy_scale_f32   x[i] *= s                              float32 logits times a constant
//   sandy_glu_clamped out[t, j] = g sigmoid(alpha g) (u + 1), g = min(a[t, j], limit), u = clamp(b[t, j], -limit, limit)
//                                                            a gated inner activation whose two halves are cut off
//   sandy_stream_add  x[t, j] += x0[t, j] + row[j]            the stream re-entering a looped span: the embedding's
//                                                            output and one learned vector join it; all float32
//   sandy_softcap_f32 x[i] = cap tanh(x[i] / cap)            float32 logits pressed into (-cap, cap)
//
// The activation is computed in 32-bit and the result rounded once.
#include "common.cuh"

namespace {

__device__ __forceinline__ float act_of(float z, int act) {
    if (act == 0) return z / (1.0f + expf(-z));                                         // silu
    if (act == 1) {                                                                     // gelu, tanh form
        const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
        return 0.5f * z * (1.0f + tanhf(u));
    }
    return z;
}

template <typename T>
__global__ void __launch_bounds__(256)
glu_kernel(const T* __restrict__ a, const T* __restrict__ b, int ld_in, T* __restrict__ out, int ld_out, int rows, int cols,
           int act) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols, j = i % cols;
        const float g = to_f32(a[t * ld_in + j]), u = to_f32(b[t * ld_in + j]);
        out[t * ld_out + j] = from_f32<T>(act_of(g, act) * u);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
cast_cols_kernel(const float* __restrict__ x, int ldx, T* __restrict__ out, int ld_out, int rows, int cols) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols, j = i % cols;
        out[t * ld_out + j] = from_f32<T>(x[t * ldx + j]);
    }
}

__global__ void __launch_bounds__(256)
scale_add_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ gain, const float* __restrict__ y2, int ldy2,
                 const float* __restrict__ gain2, float* __restrict__ x, int ldx, int rows, int cols) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols, j = i % cols;
        float branch = gain[j] * y[t * ldy + j];
        if (y2) branch += gain2[j] * y2[t * ldy2 + j];
        x[t * ldx + j] += branch;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
glu_clamped_kernel(const T* __restrict__ a, const T* __restrict__ b, int ld_in, T* __restrict__ out, int ld_out, int rows,
                   int cols, float limit, float alpha) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols, j = i % cols;
        const float g = fminf(to_f32(a[t * ld_in + j]), limit);
        const float u = fminf(fmaxf(to_f32(b[t * ld_in + j]), -limit), limit);
        out[t * ld_out + j] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

__global__ void __launch_bounds__(256)
stream_add_kernel(float* __restrict__ x, int ldx, const float* __restrict__ x0, int ldx0, const float* __restrict__ row,
                  int rows, int cols) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols, j = i % cols;
        float v = x[t * ldx + j];
        if (x0) v += x0[t * ldx0 + j];
        if (row) v += row[j];
        x[t * ldx + j] = v;
    }
}

__global__ void __launch_bounds__(256) softcap_f32_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

__global__ void __launch_bounds__(256) scale_f32_kernel(float* __restrict__ x, long long n, float s) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= s;
}

inline unsigned blocks_for(long long n) {
    const long long want = (n + 255) / 256;
    const long long cap = (long long)sandy_sm_count() * 16;
    return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

// a, b: [rows, cols] of dtype with the same pitch ld_in; out: [rows, cols] of dtype.  act: 0 silu, 1 gelu (tanh).
SANDY_API int sandy_glu(const void* a, const void* b, int ld_in, void* out, int ld_out, int rows, int cols, int act, int dtype,
                        cudaStream_t stream) {
    if (rows == 0 || cols == 0) return SANDY_OK;
    if (!a || !b || !out) return SANDY_ERR_ARGUMENT;
    const unsigned grid = blocks_for((long long)rows * cols);
    if (dtype == SANDY_F32)
        return sandy_launch(glu_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)a, (const float*)b, ld_in,
                            (float*)out, ld_out, rows, cols, act);
    if (dtype == SANDY_BF16)
        return sandy_launch(glu_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)a, (const bf16*)b, ld_in,
                            (bf16*)out, ld_out, rows, cols, act);
    return SANDY_ERR_UNSUPPORTED;
}

// x: float32 [rows, cols] with pitch ldx; out: rows of out_dtype with pitch ld_out (the caller passes the address of
// the first column to fill).
SANDY_API int sandy_cast_cols(const float* x, int ldx, void* out, int ld_out, int rows, int cols, int out_dtype,
                              cudaStream_t stream) {
    if (rows == 0 || cols == 0) return SANDY_OK;
    if (!x || !out) return SANDY_ERR_ARGUMENT;
    const unsigned grid = blocks_for((long long)rows * cols);
    if (out_dtype == SANDY_F32)
        return sandy_launch(cast_cols_kernel<float>, dim3(grid), dim3(256), 0, stream, x, ldx, (float*)out, ld_out, rows, cols);
    if (out_dtype == SANDY_BF16)
        return sandy_launch(cast_cols_kernel<bf16>, dim3(grid), dim3(256), 0, stream, x, ldx, (bf16*)out, ld_out, rows, cols);
    return SANDY_ERR_UNSUPPORTED;
}

// x [rows, cols] += gain [cols] * y [rows, cols] (+ gain2 * y2 where y2 is given: both branches of a layer whose
// sublayers read the same input are added first, then joined to the stream); all float32.
SANDY_API int sandy_scale_add(const float* y, int ldy, const float* gain, const float* y2, int ldy2, const float* gain2, float* x,
                              int ldx, int rows, int cols, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return SANDY_OK;
    if (!y || !gain || !x || (y2 && !gain2)) return SANDY_ERR_ARGUMENT;
    return sandy_launch(scale_add_kernel, dim3(blocks_for((long long)rows * cols)), dim3(256), 0, stream, y, ldy, gain, y2, ldy2,
                        gain2, x, ldx, rows, cols);
}

SANDY_API int sandy_scale_f32(float* x, long long n, float s, cudaStream_t stream) {
    if (n == 0) return SANDY_OK;
    if (!x) return SANDY_ERR_ARGUMENT;
    return sandy_launch(scale_f32_kernel, dim3(blocks_for(n)), dim3(256), 0, stream, x, n, s);
}

// a, b: [rows, cols] of dtype with the same pitch ld_in; out: [rows, cols] of dtype.  limit > 0.
SANDY_API int sandy_glu_clamped(const void* a, const void* b, int ld_in, void* out, int ld_out, int rows, int cols, float limit,
                                float alpha, int dtype, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return SANDY_OK;
    if (!a || !b || !out) return SANDY_ERR_ARGUMENT;
    if (!(limit > 0.0f)) return SANDY_ERR_UNSUPPORTED;
    const unsigned grid = blocks_for((long long)rows * cols);
    if (dtype == SANDY_F32)
        return sandy_launch(glu_clamped_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)a, (const float*)b, ld_in,
                            (float*)out, ld_out, rows, cols, limit, alpha);
    if (dtype == SANDY_BF16)
        return sandy_launch(glu_clamped_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)a, (const bf16*)b, ld_in,
                            (bf16*)out, ld_out, rows, cols, limit, alpha);
    return SANDY_ERR_UNSUPPORTED;
}

// x [rows, cols] += x0 [rows, cols] + row [cols]; x0 and row may each be null; all float32.
SANDY_API int sandy_stream_add(float* x, int ldx, const float* x0, int ldx0, const float* row, int rows, int cols,
                               cudaStream_t stream) {
    if (rows == 0 || cols == 0 || (!x0 && !row)) return SANDY_OK;
    if (!x) return SANDY_ERR_ARGUMENT;
    return sandy_launch(stream_add_kernel, dim3(blocks_for((long long)rows * cols)), dim3(256), 0, stream, x, ldx, x0, ldx0, row,
                        rows, cols);
}

SANDY_API int sandy_softcap_f32(float* x, long long n, float cap, cudaStream_t stream) {
    if (n == 0) return SANDY_OK;
    if (!x) return SANDY_ERR_ARGUMENT;
    if (!(cap > 0.0f)) return SANDY_ERR_UNSUPPORTED;
    return sandy_launch(softcap_f32_kernel, dim3(blocks_for(n)), dim3(256), 0, stream, x, n, cap);
}
