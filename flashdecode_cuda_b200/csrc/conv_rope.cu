// Row-wise kernels of mixers that pass their projections through a short causal
// convolution over time before attention:
//
//  * conv_rope_append: for every token of the step, the convolution of each q, k
//    and v channel over the token's last `taps` projected values (those of
//    earlier steps come from the sequence's state, zeros before its start), the
//    rotation of the first `rot` dimensions of every q and k head (dimension i
//    paired with i + rot/2, or, `interleaved`, dimension 2i with 2i + 1) at the
//    token's position, q to its buffer and k, v to the paged cache (value heads
//    may have a size of their own).  By option every q and k head is RMS-normed
//    (a weight vector for q and one for k, shared by the heads) between the
//    convolution and the rotation, and the values are the convolved keys as
//    they stand before that norm (no v columns in the projection then);
//  * conv_state_update: the sequence's state becomes the last taps - 1 projected
//    values after the step;
//  * gate_mul: out = a * sigmoid(g), g read with a row stride (the gate columns
//    of a packed projection);
//  * add_concat: [resid + delta | other] as one row, for a product that re-enters
//    the residual stream;
//  * relu2: y = max(x, 0)^2.
//
// The convolution, the angles' use and the sigmoid are float; storage is float
// or bfloat16.  The state is float in both.  The k-th tap multiplies the value
// taps - 1 - k steps back, and the taps are added in the order k = 0, 1, ...:
// how a prompt was cut into steps changes no bit.
#include "common.cuh"

namespace fd {

constexpr int CONV_MAX_TAPS = 8;      // more taps than this take the loop that loads one value at a time
constexpr int CONV_TPC = 8;           // tokens a CTA of a prompt step takes

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// A CTA takes one head (of q, k or v) of up to `tpc` <= CONV_TPC consecutive tokens of the step; a thread two adjacent
// channels of it (head sizes, the row length of proj and the channel count are even: 4-byte loads of bfloat16 pairs).
// What the tokens need to know - row, slot, place in the row, position, cache block - is looked up once per CTA into
// shared memory.  Then a thread convolves its channels for all of the CTA's tokens: the values its taps see are
// independent loads, issued together (a token's earlier values come from the step's own rows or, before the row's first
// new token, from the sequence's state).  The results go through shared memory to the rotation partners; after one
// barrier the thread rotates and stores q to its buffer, k and v to the paged pools.  In a step of single tokens the
// same thread also moves its channels' state on: it holds the old state in registers already.  (A thread per channel
// with its own lookups, 2-byte loads and a division by the page size per token took 75-79 us for a prompt step of
// 2,048 tokens, bound by instruction issue: 2 % of the DRAM rate under ncu.)
template <typename T>
__global__ void __launch_bounds__(128)
conv_rope_append_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w,
                        float* __restrict__ state, T* __restrict__ q_out,
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        int table_len, int rot, const int* __restrict__ tok_row,
                        const int* __restrict__ tok_pos, const int* __restrict__ row_slot,
                        const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                        T* __restrict__ k_pool, T* __restrict__ v_pool,
                        const int* __restrict__ block_table, int max_blocks, int num_blocks,
                        int block_size, int n_q, int n_kv, int d, int dv, int taps, int write_kv,
                        int update_state, int* status, int n_tok, int tpc, int interleaved,
                        const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float norm_eps,
                        int norm_count, int v_from_k) {
    extern __shared__ float y_s[];                 // [tpc][width]: the head's convolved channels of every token
    __shared__ int m_slot[CONV_TPC], m_start[CONV_TPC], m_i[CONV_TPC], m_pos[CONV_TPC], m_move[CONV_TPC];
    __shared__ float ss_s[CONV_TPC][4];            // per token and warp: the sum of squares of the head's channels
    __shared__ long long m_dst[CONV_TPC];          // element offset of the token's key or value row of this head, or -1
    const int hu = blockIdx.y;                     // head unit: q heads, then k heads, then v heads
    const int t0 = blockIdx.x * tpc;
    const int nt = min(tpc, n_tok - t0);
    const int C = (n_q + n_kv) * d + (v_from_k ? 0 : n_kv * dv);
    const bool is_q = hu < n_q, is_v = hu >= n_q + n_kv;
    const int width = is_v ? dv : d;
    const float* norm_w = is_q ? q_norm_w : (is_v ? nullptr : k_norm_w);
    const int c0 = is_v ? (n_q + n_kv) * d + (hu - n_q - n_kv) * dv : hu * d;     // the head's first channel
    const int hist = taps - 1;

    if (threadIdx.x < nt) {
        const int tt = threadIdx.x, t = t0 + tt;
        const int r = tok_row[t];
        const int slot = row_slot[r];
        const int q_start = row_q_start[r];
        const int pos = tok_pos[t];
        m_slot[tt] = slot; m_start[tt] = q_start; m_i[tt] = t - q_start; m_pos[tt] = pos;
        m_move[tt] = update_state && state != nullptr && slot >= 0 && row_q_len[r] == 1;
        long long dst = -1;
        if (slot >= 0) {
            if (rot > 0 && (pos < 0 || pos >= table_len) && hu == 0) set_status(status, STATUS_BAD_POSITION);
            if (!is_q && write_kv && pos >= 0) {
                const int col = pos / block_size;
                const int blk = col < max_blocks ? block_table[(size_t)slot * max_blocks + col] : -1;
                if (blk < 0 || blk >= num_blocks) set_status(status, STATUS_BAD_BLOCK);
                else dst = (((long long)blk * n_kv + (is_v ? hu - n_q - n_kv : hu - n_q)) * block_size + (pos - col * block_size)) * width;
            }
        }
        m_dst[tt] = dst;
    }
    __syncthreads();

    const int j = threadIdx.x * 2;                 // this thread's channels of the head: j, j + 1
    const bool active = j < width;
    const int c = c0 + (active ? j : 0);
    float y0[CONV_TPC], y1[CONV_TPC];
    if (taps <= CONV_MAX_TAPS) {
        float w0[CONV_MAX_TAPS], w1[CONV_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < CONV_MAX_TAPS; ++k) {
            w0[k] = (active && k < taps) ? conv_w[(size_t)c * taps + k] : 0.f;
            w1[k] = (active && k < taps) ? conv_w[(size_t)(c + 1) * taps + k] : 0.f;
        }
#pragma unroll
        for (int tt = 0; tt < CONV_TPC; ++tt) {
            y0[tt] = y1[tt] = 0.f;
            if (tt >= nt || !active) continue;
            const int slot = m_slot[tt];
            if (slot < 0) continue;                // padding row
            const int q_start = m_start[tt], i = m_i[tt];
            float* st = state != nullptr ? state + (size_t)slot * hist * C + c : nullptr;
            float2 u[CONV_MAX_TAPS];
#pragma unroll
            for (int k = 0; k < CONV_MAX_TAPS; ++k) {
                u[k] = make_float2(0.f, 0.f);
                if (k < taps) {
                    const int m = i - hist + k;    // index among the row's new tokens of the value this tap sees
                    if (m >= 0) u[k] = load2(proj + (size_t)(q_start + m) * ld + c);
                    else if (st != nullptr) u[k] = *reinterpret_cast<const float2*>(st + (size_t)(hist + m) * C);
                }
            }
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int k = 0; k < CONV_MAX_TAPS; ++k)
                if (k < taps) { a0 = fmaf(w0[k], u[k].x, a0); a1 = fmaf(w1[k], u[k].y, a1); }
            y0[tt] = a0; y1[tt] = a1;
            if (m_move[tt]) {                      // i == 0: u[0 .. hist-1] is the old state, u[hist] this token's value
#pragma unroll
                for (int k = 0; k < CONV_MAX_TAPS - 1; ++k)
                    if (k < hist) *reinterpret_cast<float2*>(st + (size_t)k * C) = u[k + 1];
            }
        }
    } else {
        for (int tt = 0; tt < CONV_TPC; ++tt) {
            y0[tt] = y1[tt] = 0.f;
            if (tt >= nt || !active) continue;
            const int slot = m_slot[tt];
            if (slot < 0) continue;
            const int q_start = m_start[tt], i = m_i[tt];
            float* st = state != nullptr ? state + (size_t)slot * hist * C + c : nullptr;
            float a0 = 0.f, a1 = 0.f;
            for (int k = 0; k < taps; ++k) {
                const int m = i - hist + k;
                float2 u = make_float2(0.f, 0.f);
                if (m >= 0) u = load2(proj + (size_t)(q_start + m) * ld + c);
                else if (st != nullptr) u = *reinterpret_cast<const float2*>(st + (size_t)(hist + m) * C);
                a0 = fmaf(conv_w[(size_t)c * taps + k], u.x, a0);
                a1 = fmaf(conv_w[(size_t)(c + 1) * taps + k], u.y, a1);
            }
            y0[tt] = a0; y1[tt] = a1;
            if (m_move[tt]) {
                for (int s = 0; s + 1 < hist; ++s)
                    *reinterpret_cast<float2*>(st + (size_t)s * C) = *reinterpret_cast<const float2*>(st + (size_t)(s + 1) * C);
                *reinterpret_cast<float2*>(st + (size_t)(hist - 1) * C) = load2(proj + (size_t)(t0 + tt) * ld + c);
            }
        }
    }
    if (active) {
#pragma unroll
        for (int tt = 0; tt < CONV_TPC; ++tt)
            if (tt < nt) { y_s[tt * width + j] = y0[tt]; y_s[tt * width + j + 1] = y1[tt]; }
    }
    if (norm_w != nullptr) {                       // every thread: the warps' sums are added in warp order below
#pragma unroll
        for (int tt = 0; tt < CONV_TPC; ++tt) {
            if (tt >= nt) continue;
            const float s = warp_sum(y0[tt] * y0[tt] + y1[tt] * y1[tt]);
            if ((threadIdx.x & 31) == 0) ss_s[tt][threadIdx.x >> 5] = s;
        }
    }
    __syncthreads();
    if (!active) return;

    const int half = rot >> 1;
    const int n_warps = blockDim.x >> 5;
    float nw[2] = {1.f, 1.f};
    if (norm_w != nullptr) { nw[0] = norm_w[j]; nw[1] = norm_w[j + 1]; }
#pragma unroll
    for (int tt = 0; tt < CONV_TPC; ++tt) {
        if (tt >= nt || m_slot[tt] < 0) continue;
        const int pos = m_pos[tt];
        if (v_from_k && !is_q && m_dst[tt] >= 0)   // the values: the convolved keys before norm and rotation
            store2(v_pool + m_dst[tt] + j, y0[tt], y1[tt]);
        float rinv = 1.f;
        if (norm_w != nullptr) {
            float total = 0.f;
            for (int w = 0; w < n_warps; ++w) total += ss_s[tt][w];
            rinv = rsqrtf(total / (float)norm_count + norm_eps);
        }
        const float n0 = y0[tt] * rinv * nw[0], n1 = y1[tt] * rinv * nw[1];
        float v[2] = {n0, n1};
        if (!is_v && j < rot && pos >= 0 && pos < table_len) {      // q and k heads: rotate the leading `rot` dimensions
            const float* cs = cos_t + (size_t)pos * half;
            const float* sn = sin_t + (size_t)pos * half;
            if (interleaved) {                     // the pair is this thread's own two channels
                const float c = cs[j >> 1], sv = sn[j >> 1];
                v[0] = n0 * c - n1 * sv;
                v[1] = n1 * c + n0 * sv;
            } else {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int je = j + e;
                    if (je >= rot) continue;
                    const int pj = je < half ? je + half : je - half;        // the rotation partner, normed like this one
                    const float other = y_s[tt * width + pj] * (norm_w != nullptr ? rinv * norm_w[pj] : 1.f);
                    if (je < half) v[e] = v[e] * cs[je] - other * sn[je];
                    else v[e] = v[e] * cs[je - half] + other * sn[je - half];
                }
            }
        }
        if (is_q) {
            store2(q_out + (size_t)(t0 + tt) * n_q * d + c0 + j, v[0], v[1]);
        } else if (m_dst[tt] >= 0) {
            store2((is_v ? v_pool : k_pool) + m_dst[tt] + j, v[0], v[1]);
        }
    }
}

// state[slot][s] <- the value (taps - 1 - s) places before the end of the row after this step: one of the step's
// projected values, or an older entry of the state itself (read before this thread overwrites it: s ascends and the
// source index s + q_len lies above s).
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, int ld, float* __restrict__ state,
                                         const int* __restrict__ row_slot, const int* __restrict__ row_q_start,
                                         const int* __restrict__ row_q_len, int C, int hist) {
    const int r = blockIdx.y;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int q_start = row_q_start[r], q_len = row_q_len[r];
    float* sw = state + (size_t)slot * hist * C;
    for (int s = 0; s < hist; ++s) {
        const int m = q_len - hist + s;
        sw[(size_t)s * C + c] = m >= 0 ? to_float(proj[(size_t)(q_start + m) * ld + c]) : sw[(size_t)(s + q_len) * C + c];
    }
}

template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ a, const T* __restrict__ g, int ldg, T* __restrict__ out,
                                int C, size_t total) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < total; e += stride) {
        const size_t m = e / C;
        const int c = (int)(e - m * C);
        const float z = to_float(g[m * ldg + c]);
        out[e] = from_float<T>(to_float(a[e]) / (1.f + expf(-z)));
    }
}

template <typename TD, typename T>
__global__ void add_concat_kernel(const TD* __restrict__ delta, float* __restrict__ resid,
                                  const float* __restrict__ other, T* __restrict__ out, int H) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = resid[t * H + i];
        if (delta != nullptr) {
            x += to_float(delta[t * H + i]);
            resid[t * H + i] = x;
        }
        out[t * 2 * H + i] = from_float<T>(x);
        out[t * 2 * H + H + i] = from_float<T>(other[t * H + i]);
    }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < total; e += stride) {
        const float v = fmaxf(to_float(x[e]), 0.f);
        out[e] = from_float<T>(v * v);
    }
}

static int grid_for(size_t total, int threads) {
    const size_t b = (total + threads - 1) / threads;
    return (int)(b < 148 * 16 ? b : 148 * 16);
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// dtype (0 float32, 1 bfloat16): type of proj, q_out and the cache.  proj [T, ld] holds q (n_q * d columns), k
// (n_kv * d) and v (n_kv * dv) side by side from column 0; conv_w [C, taps] and state [slots, taps - 1, C] are float
// (state may be null when taps == 1).  cos_t / sin_t [table_len, rot / 2] (unused when rot == 0).
// update_state != 0: rows that bring one token move their state on here; other rows need fd_conv_state_update.
// q_norm_w / k_norm_w [d] float or null: RMS norm of every q / k head after the convolution (mean over norm_count
// dimensions, the true head size where d is padded with zero channels).  v_from_k != 0: proj holds no v columns, dv == d,
// and v_pool receives the convolved keys as they are before norm and rotation.
extern "C" int fd_conv_rope_append(const void* proj, int ld, int dtype, const float* conv_w, float* state, void* q_out,
                                   const float* cos_t, const float* sin_t, int table_len, int rot,
                                   const int* tok_row, const int* tok_pos, const int* row_slot,
                                   const int* row_q_start, const int* row_q_len, void* k_pool, void* v_pool,
                                   const int* block_table, int max_blocks, int num_blocks, int block_size, int T,
                                   int n_q, int n_kv, int d, int dv, int taps, int write_kv, int update_state,
                                   int* status, int interleaved, const float* q_norm_w, const float* k_norm_w,
                                   float norm_eps, int norm_count, int v_from_k, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(n_q > 0 && n_kv > 0 && d > 0 && dv > 0 && taps >= 1 && block_size > 0, -2, "conv_rope_append: bad sizes");
    FD_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d, -2, "conv_rope_append: %d rotated dimensions of a head of %d", rot, d);
    FD_REQUIRE(taps == 1 || state != nullptr, -2, "conv_rope_append: %d taps need a state", taps);
    FD_REQUIRE(!v_from_k || dv == d, -2, "conv_rope_append: values taken from the keys have their size (%d, not %d)", d, dv);
    FD_REQUIRE((q_norm_w == nullptr && k_norm_w == nullptr) || (norm_count > 0 && norm_count <= d), -2,
               "conv_rope_append: a norm over %d of %d dimensions", norm_count, d);
    const int C = (n_q + n_kv) * d + (v_from_k ? 0 : n_kv * dv);
    FD_REQUIRE(ld >= C, -2, "conv_rope_append: rows of %d columns cannot hold %d channels", ld, C);
    const int widest = d > dv ? d : dv;
    FD_REQUIRE(widest <= 256 && n_q + 2 * n_kv <= 65535, -2, "conv_rope_append: heads of %d channels (max 256)", widest);
    FD_REQUIRE(d % 2 == 0 && dv % 2 == 0 && ld % 2 == 0 && (uintptr_t)proj % 4 == 0 && (uintptr_t)state % 8 == 0 &&
               (uintptr_t)q_out % 4 == 0 && (uintptr_t)k_pool % 4 == 0 && (uintptr_t)v_pool % 4 == 0, -2,
               "conv_rope_append: head sizes (%d, %d) and rows of proj (%d) must be even, buffers aligned for pairs", d, dv, ld);
    const int threads = (widest / 2 + 31) / 32 * 32;
    const int tpc = T > 64 ? CONV_TPC : 1;        // tokens a CTA takes
    const size_t smem = (size_t)tpc * widest * sizeof(float);
    const dim3 grid((T + tpc - 1) / tpc, n_q + (v_from_k ? 1 : 2) * n_kv);
    if (dtype == 0) {
        auto k = conv_rope_append_kernel<float>;
        return launch("conv_rope_append", k, grid, dim3(threads), smem, stream, dim3(1, 1, 1), (const float*)proj, ld,
                      conv_w, state, (float*)q_out, cos_t, sin_t, table_len, rot, tok_row, tok_pos, row_slot, row_q_start,
                      row_q_len, (float*)k_pool, (float*)v_pool, block_table, max_blocks, num_blocks, block_size, n_q,
                      n_kv, d, dv, taps, write_kv, update_state, status, T, tpc, interleaved, q_norm_w, k_norm_w, norm_eps,
                      norm_count, v_from_k);
    }
    auto k = conv_rope_append_kernel<bf16>;
    return launch("conv_rope_append", k, grid, dim3(threads), smem, stream, dim3(1, 1, 1), (const bf16*)proj, ld,
                  conv_w, state, (bf16*)q_out, cos_t, sin_t, table_len, rot, tok_row, tok_pos, row_slot, row_q_start,
                  row_q_len, (bf16*)k_pool, (bf16*)v_pool, block_table, max_blocks, num_blocks, block_size, n_q, n_kv,
                  d, dv, taps, write_kv, update_state, status, T, tpc, interleaved, q_norm_w, k_norm_w, norm_eps, norm_count,
                  v_from_k);
}

extern "C" int fd_conv_state_update(const void* proj, int ld, int dtype, float* state, const int* row_slot,
                                    const int* row_q_start, const int* row_q_len, int n_rows, int C, int taps,
                                    cudaStream_t stream) {
    if (n_rows == 0 || taps <= 1) return 0;
    FD_REQUIRE(state != nullptr && C > 0 && ld >= C, -2, "conv_state_update: bad arguments");
    FD_REQUIRE(n_rows <= 65535, -2, "conv_state_update: batch of %d rows too large", n_rows);
    dim3 grid((C + 127) / 128, n_rows);
    if (dtype == 0)
        return launch("conv_state_update", conv_state_update_kernel<float>, grid, dim3(128), 0, stream, dim3(1, 1, 1),
                      (const float*)proj, ld, state, row_slot, row_q_start, row_q_len, C, taps - 1);
    return launch("conv_state_update", conv_state_update_kernel<bf16>, grid, dim3(128), 0, stream, dim3(1, 1, 1),
                  (const bf16*)proj, ld, state, row_slot, row_q_start, row_q_len, C, taps - 1);
}

// out[m, c] = a[m, c] * sigmoid(g[m * ldg + c]) for M rows of C columns.
extern "C" int fd_gate_mul(const void* a, const void* g, int ldg, void* out, int dtype, int M, int C, cudaStream_t stream) {
    const size_t total = (size_t)M * C;
    if (total == 0) return 0;
    if (dtype == 0)
        return launch("gate_mul", gate_mul_kernel<float>, dim3(grid_for(total, 256)), dim3(256), 0, stream, dim3(1, 1, 1),
                      (const float*)a, (const float*)g, ldg, (float*)out, C, total);
    return launch("gate_mul", gate_mul_kernel<bf16>, dim3(grid_for(total, 256)), dim3(256), 0, stream, dim3(1, 1, 1),
                  (const bf16*)a, (const bf16*)g, ldg, (bf16*)out, C, total);
}

// resid += delta (delta may be null); out[t] = [resid[t] | other[t]] in the type `dtype`.
// delta_dtype: 0 float32, 1 bfloat16.
extern "C" int fd_add_concat(const void* delta, int delta_dtype, float* resid, const float* other, void* out, int dtype,
                             int T, int H, cudaStream_t stream) {
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
#define FD_AC(TD_, T_)                                                                                         \
    return launch("add_concat", add_concat_kernel<TD_, T_>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1), \
                  (const TD_*)delta, resid, other, (T_*)out, H)
    if (dtype == 0) {
        if (delta_dtype == 0) FD_AC(float, float);
        FD_AC(bf16, float);
    }
    if (delta_dtype == 0) FD_AC(float, bf16);
    FD_AC(bf16, bf16);
#undef FD_AC
}

extern "C" int fd_relu2(const void* x, void* out, int dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (dtype == 0)
        return launch("relu2", relu2_kernel<float>, dim3(grid_for((size_t)total, 256)), dim3(256), 0, stream,
                      dim3(1, 1, 1), (const float*)x, (float*)out, (size_t)total);
    return launch("relu2", relu2_kernel<bf16>, dim3(grid_for((size_t)total, 256)), dim3(256), 0, stream, dim3(1, 1, 1),
                  (const bf16*)x, (bf16*)out, (size_t)total);
}
