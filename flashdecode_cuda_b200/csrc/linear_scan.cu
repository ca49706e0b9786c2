// Linear-attention recurrences with a matrix state per head, and the per-head norm that follows them.
//
//   S_t = diag(a_t) S_(t-1) + b_t v_t^T,      o_t = S_t^T q_t          S [d, dv] per sequence and head
//
//  * mode 0 (constant decay): a_t = decay[h] for every channel, b_t = rot(k_t) * k_scale, q_t = rot(q_t); rot turns
//    the first `rot` dimensions of a head at the token's position, dimension i paired with i + rot/2.
//  * mode 1 (forget gate): a_t = f_t = lower + (1 - lower) * sigmoid(z_t) per channel, b_t = 1 - f_t,
//    q_t = silu(zq_t); z and zq are columns of the projection.
//
// The state lives in float per cache slot and is carried from step to step; a step's tokens of a sequence are walked in
// order, so the sums of every state element are the same whether a prompt comes whole, in portions or token by token.
// Everything after the projection is float: angles' use, gates, decay, state, output.
//
// A CTA of 128 threads takes one sequence of the step, one head and a tile of value columns.  DS = 4 (d <= 128) or 8
// adjacent lanes share a column and hold every DS-th row of it in registers (at most 32 each); the tokens' q, a, b
// and v are staged in shared memory a chunk at a time by all threads, then the chunk is walked token by token:
// per token a thread does two fused multiply-adds per state element it holds and the DS lanes add their partial
// outputs with shuffles.
//
//  * head_norm_gate: y = o / sqrt(mean(o^2) + eps) per token and head (over dv), times an optional weight [dv], times
//    an optional silu(gate) read from a column range of a packed projection, times a constant; written with a row
//    stride and a column offset of its own so that several mixers can fill one buffer.
#include <math.h>

#include "common.cuh"

namespace fd {

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_RPT = 32;           // state rows a thread holds at most

struct ScanParams {
    const void* proj; int ld;          // [T, ld]
    int q_col, k_col, v_col;           // first columns of q, of k (mode 0) or the gate's pre-activation (mode 1), of v
    float* state;                      // [slots, H, d, dv]
    float* out;                        // [T, H * dv]
    const float* decay;                // [H] (mode 0)
    const float* lower;                // [H * d] (mode 1)
    const float* cos_t; const float* sin_t; int table_len, rot;
    float k_scale;
    const int* row_slot; const int* row_q_start; const int* row_q_len; const int* row_ctx_len;
    int H, d, dv, mode, write_state, DS, TC;
    int* status;
};

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
linear_scan_kernel(const ScanParams p) {
    const int r = blockIdx.z, h = blockIdx.y;
    const int slot = p.row_slot[r];
    if (slot < 0) return;
    const int q_start = p.row_q_start[r], q_len = p.row_q_len[r], ctx = p.row_ctx_len[r];
    const int d = p.d, dv = p.dv, DS = p.DS, TC = p.TC;
    const int VT = SCAN_THREADS / DS;
    const int tid = threadIdx.x;
    const int vl = tid / DS, ds = tid - vl * DS;
    const int v = blockIdx.x * VT + vl;
    const bool v_ok = v < dv;

    extern __shared__ float sm[];
    float* q_s = sm;                    // [TC][d]
    float* b_s = q_s + TC * d;          // [TC][d]
    float* a_s = b_s + TC * d;          // [TC][d] (mode 1)
    float* v_s = a_s + (p.mode ? TC * d : 0);   // [TC][VT]

    const T* proj = static_cast<const T*>(p.proj);
    float* st = p.state + ((size_t)slot * p.H + h) * d * dv;
    float S[SCAN_RPT];
#pragma unroll
    for (int ii = 0; ii < SCAN_RPT; ++ii) {
        const int i = ii * DS + ds;
        S[ii] = (i < d && v_ok) ? st[(size_t)i * dv + v] : 0.f;
    }
    const float g = p.mode == 0 ? p.decay[h] : 0.f;
    const int half = p.rot >> 1;

    for (int c0 = 0; c0 < q_len; c0 += TC) {
        const int n = min(TC, q_len - c0);
        __syncthreads();
        for (int idx = tid; idx < n * d; idx += SCAN_THREADS) {
            const int tt = idx / d, i = idx - tt * d;
            const size_t row = (size_t)(q_start + c0 + tt) * p.ld;
            const float xq = to_float(proj[row + p.q_col + h * d + i]);
            const float xk = to_float(proj[row + p.k_col + h * d + i]);
            if (p.mode == 0) {
                float qv = xq, kv = xk;
                if (i < p.rot) {
                    const int pos = ctx + c0 + tt;
                    if (pos < p.table_len) {
                        const bool first = i < half;
                        const int pi = first ? i : i - half;
                        const int partner = first ? i + half : i - half;
                        const float c = p.cos_t[(size_t)pos * half + pi], s = p.sin_t[(size_t)pos * half + pi];
                        const float yq = to_float(proj[row + p.q_col + h * d + partner]);
                        const float yk = to_float(proj[row + p.k_col + h * d + partner]);
                        qv = first ? xq * c - yq * s : xq * c + yq * s;
                        kv = first ? xk * c - yk * s : xk * c + yk * s;
                    } else if (i == 0 && h == 0 && blockIdx.x == 0) {
                        set_status(p.status, STATUS_BAD_POSITION);
                    }
                }
                q_s[idx] = qv;
                b_s[idx] = kv * p.k_scale;
            } else {
                const float lo = p.lower[h * d + i];
                const float f = lo + (1.f - lo) / (1.f + expf(-xk));
                q_s[idx] = xq / (1.f + expf(-xq));
                a_s[idx] = f;
                b_s[idx] = 1.f - f;
            }
        }
        for (int idx = tid; idx < n * VT; idx += SCAN_THREADS) {
            const int tt = idx / VT, c = idx - tt * VT;
            const int vc = blockIdx.x * VT + c;
            v_s[idx] = vc < dv ? to_float(proj[(size_t)(q_start + c0 + tt) * p.ld + p.v_col + h * dv + vc]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float vv = v_s[tt * VT + vl];
            const float* qr = q_s + tt * d;
            const float* br = b_s + tt * d;
            const float* ar = a_s + tt * d;
            float o = 0.f;
            if (p.mode == 0) {
#pragma unroll
                for (int ii = 0; ii < SCAN_RPT; ++ii) {
                    if (ii * DS >= d) break;
                    const int i = ii * DS + ds;
                    if (i < d) {
                        S[ii] = fmaf(g, S[ii], br[i] * vv);
                        o = fmaf(S[ii], qr[i], o);
                    }
                }
            } else {
#pragma unroll
                for (int ii = 0; ii < SCAN_RPT; ++ii) {
                    if (ii * DS >= d) break;
                    const int i = ii * DS + ds;
                    if (i < d) {
                        S[ii] = fmaf(ar[i], S[ii], br[i] * vv);
                        o = fmaf(S[ii], qr[i], o);
                    }
                }
            }
            for (int off = 1; off < DS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (ds == 0 && v_ok) p.out[(size_t)(q_start + c0 + tt) * p.H * dv + h * dv + v] = o;
        }
    }
    if (p.write_state && v_ok) {
#pragma unroll
        for (int ii = 0; ii < SCAN_RPT; ++ii) {
            const int i = ii * DS + ds;
            if (i < d) st[(size_t)i * dv + v] = S[ii];
        }
    }
}

// A warp per (token, head).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ gate,
                                      int ldg, T* __restrict__ out, int ld_out, int n_pairs, int H, int dv, float eps,
                                      float scale) {
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= n_pairs) return;
    const int lane = threadIdx.x & 31;
    const int t = pair / H, h = pair - t * H;
    const float* x = o + (size_t)t * H * dv + (size_t)h * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(x[j], x[j], ss);
    ss = warp_sum(ss);
    const float rs = scale / sqrtf(ss / (float)dv + eps);
    for (int j = lane; j < dv; j += 32) {
        float y = x[j] * rs;
        if (w != nullptr) y *= w[j];
        if (gate != nullptr) {
            const float z = to_float(gate[(size_t)t * ldg + h * dv + j]);
            y *= z / (1.f + expf(-z));
        }
        out[(size_t)t * ld_out + h * dv + j] = from_float<T>(y);
    }
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// proj [T, ld] of `dtype` (0 float32, 1 bfloat16) holds q at q_col, k (mode 0) or the gate's pre-activation (mode 1)
// at k_col - H * d columns each - and v at v_col (H * dv columns).  state [slots, H, d, dv] and out [T, H * dv] float.
// mode 0: decay [H], cos_t / sin_t [table_len, rot / 2] (unused when rot == 0), k_scale.  mode 1: lower [H * d].
extern "C" int fd_linear_scan(const void* proj, int ld, int dtype, int q_col, int k_col, int v_col, float* state,
                              float* out, int mode, const float* decay, const float* lower, const float* cos_t,
                              const float* sin_t, int table_len, int rot, float k_scale, const int* row_slot,
                              const int* row_q_start, const int* row_q_len, const int* row_ctx_len, int n_rows, int H,
                              int d, int dv, int write_state, int* status, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    FD_REQUIRE(H > 0 && d > 0 && dv > 0 && d <= 8 * SCAN_RPT, -2, "linear_scan: %d heads of %d x %d (d at most %d)", H, d,
               dv, 8 * SCAN_RPT);
    FD_REQUIRE(mode == 0 || mode == 1, -2, "linear_scan: unknown mode %d", mode);
    FD_REQUIRE(mode == 1 ? lower != nullptr : decay != nullptr, -2, "linear_scan: the mode's constants are missing");
    FD_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d && (rot == 0 || mode == 1 || (cos_t && sin_t)), -2,
               "linear_scan: %d rotated dimensions of %d", rot, d);
    FD_REQUIRE(n_rows <= 65535 && H <= 65535, -2, "linear_scan: %d rows, %d heads", n_rows, H);
    ScanParams p;
    p.proj = proj; p.ld = ld; p.q_col = q_col; p.k_col = k_col; p.v_col = v_col; p.state = state; p.out = out;
    p.decay = decay; p.lower = lower; p.cos_t = cos_t; p.sin_t = sin_t; p.table_len = table_len;
    p.rot = mode == 0 ? rot : 0; p.k_scale = k_scale;
    p.row_slot = row_slot; p.row_q_start = row_q_start; p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len;
    p.H = H; p.d = d; p.dv = dv; p.mode = mode; p.write_state = write_state; p.status = status;
    p.DS = d <= 4 * SCAN_RPT ? 4 : 8;
    p.TC = d <= 128 ? 16 : 8;
    const int VT = SCAN_THREADS / p.DS;
    const size_t smem = (size_t)((mode ? 3 : 2) * p.TC * d + p.TC * VT) * sizeof(float);
    const dim3 grid((dv + VT - 1) / VT, H, n_rows);
    if (dtype == 0)
        return launch("linear_scan", linear_scan_kernel<float>, grid, dim3(SCAN_THREADS), smem, stream, dim3(1, 1, 1), p);
    return launch("linear_scan", linear_scan_kernel<bf16>, grid, dim3(SCAN_THREADS), smem, stream, dim3(1, 1, 1), p);
}

// o [T, H * dv] float; w [dv] float or null; gate: pointer to the first gate column of a packed projection with row
// stride ldg (dtype as out), or null; out: pointer to the first output column, row stride ld_out.
extern "C" int fd_head_norm_gate(const float* o, const float* w, const void* gate, int ldg, void* out, int ld_out,
                                 int dtype, int T, int H, int dv, float eps, float scale, cudaStream_t stream) {
    const long long pairs = (long long)T * H;
    if (pairs == 0) return 0;
    FD_REQUIRE(pairs < (1ll << 31) - 8, -2, "head_norm_gate: too many rows");
    const dim3 grid((unsigned)((pairs + 3) / 4));
    if (dtype == 0)
        return launch("head_norm_gate", head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, dim3(1, 1, 1), o, w,
                      (const float*)gate, ldg, (float*)out, ld_out, (int)pairs, H, dv, eps, scale);
    return launch("head_norm_gate", head_norm_gate_kernel<bf16>, grid, dim3(128), 0, stream, dim3(1, 1, 1), o, w,
                  (const bf16*)gate, ldg, (bf16*)out, ld_out, (int)pairs, H, dv, eps, scale);
}
