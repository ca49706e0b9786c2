// Dynamic Tanh "norm" fused with the deferred residual add, and two small float epilogues.
//
//  * add_dyn_tanh: resid += delta; out = tanh(alpha * resid) * w + b.  No mean and no
//    variance: every element stands alone, so a row is cut over several CTAs when the step
//    has few rows.  The sum, the tanh and the affine map are float (tanhf, not the fast
//    form); w and b are float vectors, alpha a scalar passed by value.  Rows may be gathered
//    through an index list (the final norm at the wanted places).
//  * quad_exp_act: y = a_p z^2 + z/2 for z > 0, (1/2 + a_q)(exp(z) - 1 - z) + z/2 otherwise,
//    with a_p = softplus(p), a_q = softplus(q) read from a two-element tensor.
//  * scale_f32: x <- x * s in place.
//  * axpy_f32: y <- s * x (+ y) with y float and x float or bfloat16: a weighted sum of sub-layer outputs.
#include <math.h>

#include "common.cuh"

namespace fd {

constexpr int DT_THREADS = 256;
constexpr int DT_COLS = DT_THREADS * 4;        // columns of a row that one CTA takes

template <typename TD> __device__ __forceinline__ void load4(const TD* p, float f[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float f[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float f[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float f[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float f[4]) {
    uint2 v;
    *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(f[0], f[1]);
    *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(p) = v;
}

// grid (column tiles, rows).  VEC: H is a multiple of 4 and a thread takes 4 adjacent columns.
template <typename TD, typename TO, bool VEC>
__global__ void __launch_bounds__(DT_THREADS)
add_dyn_tanh_kernel(const TD* __restrict__ delta, float* __restrict__ resid, int write_resid,
                    const float* __restrict__ w, const float* __restrict__ b, float alpha, TO* __restrict__ out,
                    const int* __restrict__ rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int j = blockIdx.y;
    const int r = rows ? rows[j] : j;
    if (VEC) {
        const int i = (blockIdx.x * DT_THREADS + threadIdx.x) * 4;
        if (i >= H) return;
        float x[4], wv[4], bv[4];
        load4<float>(resid + (size_t)r * H + i, x);
        load4<float>(w + i, wv);
        load4<float>(b + i, bv);
        if (delta != nullptr) {
            float d[4];
            load4<TD>(delta + (size_t)r * H + i, d);
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] += d[e];
            if (write_resid) store4(resid + (size_t)r * H + i, x);
        }
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = fmaf(tanhf(alpha * x[e]), wv[e], bv[e]);
        store4(out + (size_t)j * H + i, y);
    } else {
        for (int i = blockIdx.x * DT_COLS + threadIdx.x; i < min(H, (int)(blockIdx.x + 1) * DT_COLS); i += DT_THREADS) {
            float x = resid[(size_t)r * H + i];
            if (delta != nullptr) {
                x += to_float(delta[(size_t)r * H + i]);
                if (write_resid) resid[(size_t)r * H + i] = x;
            }
            out[(size_t)j * H + i] = from_float<TO>(fmaf(tanhf(alpha * x), w[i], b[i]));
        }
    }
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void quad_exp_act_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ pq, size_t total) {
    const float ap = softplus_f(pq[0]), aq = 0.5f + softplus_f(pq[1]);
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < total; e += stride) {
        const float z = to_float(x[e]);
        const float y = z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
        out[e] = from_float<T>(y);
    }
}

__global__ void scale_f32_kernel(float* __restrict__ x, size_t n, float s) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < n; e += stride) x[e] *= s;
}

template <typename T>
__global__ void axpy_f32_kernel(float* __restrict__ y, const T* __restrict__ x, size_t n, float s, int accumulate) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < n; e += stride) y[e] = accumulate ? fmaf(s, to_float(x[e]), y[e]) : s * to_float(x[e]);
}

static unsigned blocks_for(size_t total, int threads) {
    const size_t b = (total + threads - 1) / threads;
    return (unsigned)(b < 148 * 16 ? b : 148 * 16);
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// delta (dtype delta_dtype: 0 float32, 1 bfloat16; may be null) and resid [*, H]; out [n_out, H] of out_dtype;
// rows (optional) [n_out] gathers; w, b float [H].
extern "C" int fd_add_dyn_tanh(const void* delta, int delta_dtype, float* resid, int write_resid, const float* w,
                               const float* b, float alpha, void* out, int out_dtype, const int* rows, int n_out, int H,
                               cudaStream_t stream) {
    if (n_out == 0 || H == 0) return 0;
    FD_REQUIRE(n_out <= 65535 * 32, -2, "add_dyn_tanh: %d rows", n_out);
    const bool vec = H % 4 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)b % 16 == 0 &&
                     (uintptr_t)out % 16 == 0 && (uintptr_t)delta % 16 == 0;
    const dim3 grid((H + DT_COLS - 1) / DT_COLS, n_out);
    FD_REQUIRE(grid.y <= 65535, -2, "add_dyn_tanh: %d rows exceed one launch", n_out);
#define FD_DT(TD_, TO_)                                                                                             \
    do {                                                                                                            \
        if (vec)                                                                                                    \
            return launch("add_dyn_tanh", add_dyn_tanh_kernel<TD_, TO_, true>, grid, dim3(DT_THREADS), 0, stream,  \
                          dim3(1, 1, 1), (const TD_*)delta, resid, write_resid, w, b, alpha, (TO_*)out, rows, H);   \
        return launch("add_dyn_tanh", add_dyn_tanh_kernel<TD_, TO_, false>, grid, dim3(DT_THREADS), 0, stream,     \
                      dim3(1, 1, 1), (const TD_*)delta, resid, write_resid, w, b, alpha, (TO_*)out, rows, H);       \
    } while (0)
    if (out_dtype == 0) {
        if (delta_dtype == 0) FD_DT(float, float);
        FD_DT(bf16, float);
    }
    if (delta_dtype == 0) FD_DT(float, bf16);
    FD_DT(bf16, bf16);
#undef FD_DT
}

extern "C" int fd_quad_exp_act(const void* x, void* out, int dtype, const float* pq, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (dtype == 0)
        return launch("quad_exp_act", quad_exp_act_kernel<float>, dim3(blocks_for((size_t)total, 256)), dim3(256), 0,
                      stream, dim3(1, 1, 1), (const float*)x, (float*)out, pq, (size_t)total);
    return launch("quad_exp_act", quad_exp_act_kernel<bf16>, dim3(blocks_for((size_t)total, 256)), dim3(256), 0, stream,
                  dim3(1, 1, 1), (const bf16*)x, (bf16*)out, pq, (size_t)total);
}

extern "C" int fd_scale_f32(float* x, long long n, float s, cudaStream_t stream) {
    if (n <= 0) return 0;
    return launch("scale_f32", scale_f32_kernel, dim3(blocks_for((size_t)n, 256)), dim3(256), 0, stream, dim3(1, 1, 1),
                  x, (size_t)n, s);
}

// y [n] float <- s * x (+ y when accumulate); x of `dtype` (0 float32, 1 bfloat16).
extern "C" int fd_axpy_f32(float* y, const void* x, int dtype, long long n, float s, int accumulate, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == 0)
        return launch("axpy_f32", axpy_f32_kernel<float>, dim3(blocks_for((size_t)n, 256)), dim3(256), 0, stream,
                      dim3(1, 1, 1), y, (const float*)x, (size_t)n, s, accumulate);
    return launch("axpy_f32", axpy_f32_kernel<bf16>, dim3(blocks_for((size_t)n, 256)), dim3(256), 0, stream,
                  dim3(1, 1, 1), y, (const bf16*)x, (size_t)n, s, accumulate);
}
