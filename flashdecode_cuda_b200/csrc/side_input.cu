// What a layer adds to the residual stream from the token itself (a second, narrow embedding table gated by the stream),
// and a vector added to the whole stream between layers.
//
//   x    = resid + dscale * delta                      the stream as it stands once the pending output is added (kept)
//   g    = gelu_tanh(G x) * e                          G [dim, H]; e = side_table[token, col0 .. col0 + dim)
//   y    = P g                                         P [H, dim]
//   out  = y / sqrt(mean(y^2) + eps) * w               float, still to be added to the stream by whoever norms next
//
//  * add_cast: x as above, written back to resid and, rounded once, to a matrix for the product with G;
//  * side_gate_mul: g from z = G x (float) and the table row of every token;
//  * token_side_row: all of it in two launches for steps of few tokens.  The first takes a CTA per token and eight
//    rows of G, a warp per row (lanes over k, 16-byte loads), so that a step of eight tokens still spreads over
//    dozens of SMs; the second a CTA per token, a thread per row of P, then the norm.  Every sum has one fixed order per
//    output whatever else the step holds;
//  * add_row_vector: resid <- resid + dscale * delta + vec.
//
// The sums, the activation and the norm are float; G, P and the table are float or bfloat16.
#include <math.h>

#include "common.cuh"

namespace fd {

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TD, typename T>
__global__ void add_cast_kernel(const TD* __restrict__ delta, float* __restrict__ resid, T* __restrict__ out, int H,
                                float dscale) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = resid[t * H + i];
        if (delta != nullptr) {
            x = fmaf(dscale, to_float(delta[t * H + i]), x);
            resid[t * H + i] = x;
        }
        out[t * H + i] = from_float<T>(x);
    }
}

template <typename T>
__global__ void side_gate_mul_kernel(const float* __restrict__ z, const int* __restrict__ tokens,
                                     const T* __restrict__ table, int ld_table, int col0, int V, T* __restrict__ g,
                                     int dim, size_t total, int* status) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < total; e += stride) {
        const size_t t = e / dim;
        const int j = (int)(e - t * dim);
        const int id = tokens[t];
        float v = 0.f;
        if (id < 0 || id >= V) set_status(status, STATUS_BAD_TOKEN);
        else v = gelu_tanh_f(z[e]) * to_float(table[(size_t)id * ld_table + col0 + j]);
        g[e] = from_float<T>(v);
    }
}

// First launch of the form for few tokens: a CTA per token and group of eight gate outputs, a warp per output.  Every CTA
// forms the token's row of x in shared memory (the stream is not written here: the CTAs of a token would race).
template <typename TD, typename T>
__global__ void __launch_bounds__(256)
token_side_gate_kernel(const TD* __restrict__ delta, const float* __restrict__ resid, float dscale,
                       const int* __restrict__ tokens, const T* __restrict__ table, int ld_table, int col0, int V,
                       const T* __restrict__ G, float* __restrict__ g_out, int H, int dim, int* status) {
    extern __shared__ __align__(16) float x_s[];   // [H]
    const size_t t = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int o = blockIdx.x * 8 + warp;
    constexpr int VEC = 16 / sizeof(T);
    const bool vec = H % VEC == 0 && (uintptr_t)G % 16 == 0;
    // this warp's first weights are on their way before the row is there
    uint4 first = make_uint4(0, 0, 0, 0);
    if (vec && o < dim && lane < H / VEC) first = *reinterpret_cast<const uint4*>(G + (size_t)o * H + lane * VEC);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = resid[t * H + i];
        if (delta != nullptr) x = fmaf(dscale, to_float(delta[t * H + i]), x);
        x_s[i] = to_float(from_float<T>(x));       // the product's operand in the model's dtype, as the other path rounds it
    }
    __syncthreads();
    if (o >= dim) return;
    const int id = tokens[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && lane == 0 && blockIdx.x == 0) set_status(status, STATUS_BAD_TOKEN);
    const T* gr = G + (size_t)o * H;
    float acc = 0.f;
    if (vec) {
        for (int c0 = lane; c0 < H / VEC; c0 += 4 * 32) {          // four 16-byte loads of the row in flight together
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * 32;
                if (c < H / VEC) raw[u] = c == lane ? first : *reinterpret_cast<const uint4*>(gr + c * VEC);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * 32;
                if (c >= H / VEC) continue;
                const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc = fmaf(to_float(e[j]), x_s[c * VEC + j], acc);
            }
        }
    } else {
        for (int k = lane; k < H; k += 32) acc = fmaf(to_float(gr[k]), x_s[k], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        const float e = ok ? to_float(table[(size_t)id * ld_table + col0 + o]) : 0.f;
        g_out[t * dim + o] = to_float(from_float<T>(gelu_tanh_f(acc) * e));
    }
}

// Second launch: a CTA per token.  It writes the completed stream back, multiplies the token's gate values by P (a
// thread per row of P, 16-byte loads where the rows allow them), norms the result and writes the contribution.
template <typename TD, typename T, typename TW>
__global__ void __launch_bounds__(1024)
token_side_proj_kernel(const TD* __restrict__ delta, float* __restrict__ resid, float dscale,
                       const float* __restrict__ g_in, const T* __restrict__ P, const TW* __restrict__ w, float eps,
                       float* __restrict__ out, int H, int dim) {
    extern __shared__ __align__(16) float sm[];
    float* y_s = sm;                               // [H]
    float* g_s = y_s + ((H + 3) & ~3);             // [dim]
    float* red = g_s + ((dim + 3) & ~3);           // [33]
    const size_t t = blockIdx.x;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int AHEAD = 4;                       // 16-byte loads of a row in flight together
    const bool vec = dim % VEC == 0 && (uintptr_t)P % 16 == 0;
    // the first loads of this thread's first row need nothing but P: they are on their way while g arrives
    uint4 first[AHEAD];
    if (vec && threadIdx.x < H) {
#pragma unroll
        for (int u = 0; u < AHEAD; ++u)
            if (u < dim / VEC) first[u] = *reinterpret_cast<const uint4*>(P + (size_t)threadIdx.x * dim + u * VEC);
    }
    for (int j = threadIdx.x; j < dim; j += blockDim.x) g_s[j] = g_in[t * dim + j];
    if (delta != nullptr)
        for (int i = threadIdx.x; i < H; i += blockDim.x)
            resid[t * H + i] = fmaf(dscale, to_float(delta[t * H + i]), resid[t * H + i]);
    __syncthreads();
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const T* pr = P + (size_t)i * dim;
        float acc = 0.f;
        if (vec) {
            for (int c0 = 0; c0 < dim / VEC; c0 += AHEAD) {
                uint4 raw[AHEAD];
#pragma unroll
                for (int u = 0; u < AHEAD; ++u)
                    if (c0 + u < dim / VEC)
                        raw[u] = (c0 == 0 && i == threadIdx.x) ? first[u] : *reinterpret_cast<const uint4*>(pr + (c0 + u) * VEC);
#pragma unroll
                for (int u = 0; u < AHEAD; ++u) {
                    if (c0 + u >= dim / VEC) continue;
                    const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) acc = fmaf(to_float(e[j]), g_s[(c0 + u) * VEC + j], acc);
                }
            }
        } else {
            for (int j = 0; j < dim; ++j) acc = fmaf(to_float(pr[j]), g_s[j], acc);
        }
        y_s[i] = acc;
        ss += acc * acc;
    }
    const float total = block_sum(ss, red);
    const float rstd = rsqrtf(total / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[t * H + i] = y_s[i] * rstd * to_float(w[i]);
}

template <typename TD>
__global__ void add_row_vector_kernel(const TD* __restrict__ delta, float* __restrict__ resid,
                                      const float* __restrict__ vec, int H, float dscale) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = resid[t * H + i];
        if (delta != nullptr) x = fmaf(dscale, to_float(delta[t * H + i]), x);
        resid[t * H + i] = x + vec[i];
    }
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// resid [T, H] float += dscale * delta (delta [T, H] of delta_dtype, or null); out [T, H] of `dtype` = the sum, rounded.
extern "C" int fd_add_cast(const void* delta, int delta_dtype, float* resid, void* out, int dtype, int T, int H,
                           float dscale, cudaStream_t stream) {
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
#define FD_ACAST(TD_, T_)                                                                                    \
    return launch("add_cast", add_cast_kernel<TD_, T_>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1), \
                  (const TD_*)delta, resid, (T_*)out, H, dscale)
    if (dtype == 0) {
        if (delta_dtype == 0) FD_ACAST(float, float);
        FD_ACAST(bf16, float);
    }
    if (delta_dtype == 0) FD_ACAST(float, bf16);
    FD_ACAST(bf16, bf16);
#undef FD_ACAST
}

// g [T, dim] of `dtype` = gelu_tanh(z [T, dim] float) * table[tokens[t], col0 .. col0 + dim); table [V, ld_table].
extern "C" int fd_side_gate_mul(const float* z, const int* tokens, const void* table, int ld_table, int col0, int V,
                                void* g, int dtype, int T, int dim, int* status, cudaStream_t stream) {
    const size_t total = (size_t)T * dim;
    if (total == 0) return 0;
    FD_REQUIRE(col0 >= 0 && col0 + dim <= ld_table, -2, "side_gate_mul: columns %d .. %d of a table of %d", col0, col0 + dim, ld_table);
    const size_t want = (total + 255) / 256;
    const dim3 grid((unsigned)(want < 148 * 16 ? want : 148 * 16));
    if (dtype == 0)
        return launch("side_gate_mul", side_gate_mul_kernel<float>, grid, dim3(256), 0, stream, dim3(1, 1, 1), z, tokens,
                      (const float*)table, ld_table, col0, V, (float*)g, dim, total, status);
    return launch("side_gate_mul", side_gate_mul_kernel<bf16>, grid, dim3(256), 0, stream, dim3(1, 1, 1), z, tokens,
                  (const bf16*)table, ld_table, col0, V, (bf16*)g, dim, total, status);
}

// The whole contribution in two launches for steps of few tokens; out [T, H] float, g [T, dim] float scratch.  G [dim, H],
// P [H, dim] and the table of `dtype`; w [H] of w_dtype.  Returns -2 for sizes whose rows do not fit the shared memory
// (the caller takes the path of separate kernels).
extern "C" int fd_token_side_row(const void* delta, int delta_dtype, float* resid, float dscale, const int* tokens,
                                 const void* table, int ld_table, int col0, int V, const void* G, const void* P,
                                 const void* w, int w_dtype, float eps, float* g, float* out, int dtype, int T, int H,
                                 int dim, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(col0 >= 0 && col0 + dim <= ld_table && dim > 0 && H > 0 && T <= 65535, -2, "token_side_row: bad sizes");
    const size_t smem1 = (size_t)((H + 3) & ~3) * sizeof(float);
    const size_t smem2 = (((H + 3) & ~3) + ((dim + 3) & ~3) + 40) * sizeof(float);
    FD_REQUIRE(smem2 <= 48 * 1024, -2, "token_side_row: a row of %d and %d gate values need %zu bytes of shared memory", H, dim, smem2);
    const dim3 grid1((dim + 7) / 8, T), grid2(T), block(256), one(1, 1, 1);
    const dim3 block2(H >= 1024 ? 1024 : (H >= 512 ? 512 : 256));
#define FD_TSR(TD_, T_, TW_)                                                                                          \
    do {                                                                                                              \
        int rc = launch("token_side_gate", token_side_gate_kernel<TD_, T_>, grid1, block, smem1, stream, one,         \
                        (const TD_*)delta, (const float*)resid, dscale, tokens, (const T_*)table, ld_table, col0, V,  \
                        (const T_*)G, g, H, dim, status);                                                             \
        if (rc != 0) return rc;                                                                                       \
        return launch("token_side_proj", token_side_proj_kernel<TD_, T_, TW_>, grid2, block2, smem2, stream, one,      \
                      (const TD_*)delta, resid, dscale, (const float*)g, (const T_*)P, (const TW_*)w, eps, out, H, dim); \
    } while (0)
    if (dtype == 0) {
        FD_REQUIRE(w_dtype == 0, -2, "token_side_row: the float path takes float weights");
        if (delta_dtype == 0) FD_TSR(float, float, float);
        FD_TSR(bf16, float, float);
    }
    if (w_dtype == 0) {
        if (delta_dtype == 0) FD_TSR(float, bf16, float);
        FD_TSR(bf16, bf16, float);
    }
    if (delta_dtype == 0) FD_TSR(float, bf16, bf16);
    FD_TSR(bf16, bf16, bf16);
#undef FD_TSR
}

// resid [T, H] float <- resid + dscale * delta + vec (delta [T, H] of delta_dtype or null; vec [H] float).
extern "C" int fd_add_row_vector(const void* delta, int delta_dtype, float* resid, const float* vec, int T, int H,
                                 float dscale, cudaStream_t stream) {
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (delta_dtype == 0)
        return launch("add_row_vector", add_row_vector_kernel<float>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                      (const float*)delta, resid, vec, H, dscale);
    return launch("add_row_vector", add_row_vector_kernel<bf16>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                  (const bf16*)delta, resid, vec, H, dscale);
}
