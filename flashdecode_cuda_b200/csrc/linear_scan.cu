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
// Long portions (prompts) are cut into segments of `seg_len` tokens that run side by side, in three launches:
//  1. every segment but a sequence's last walks its tokens from a zero state and leaves U = its own contribution to
//     the state [d, dv] and, with a forget gate, the product A of its gates per channel (a constant decay's product is
//     decay^seg_len);
//  2. per sequence, head and state element the segments are chained: S_0 = the cached state, S_(s+1) = A_s S_s + U_s;
//  3. every segment walks its tokens again from its S_s and writes the outputs; the last one writes the state back.
// The recurrence itself is unchanged, so nothing is divided by a product of gates that could vanish.
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
    // segments: phase 0 = the whole portion in one CTA; 1 = a segment from a zero state, leaves U (and A); 3 = a segment
    // from its chained start state, writes outputs.  seg_state [segment slots, H, d, dv], seg_decay [segment slots, H, d].
    int phase, seg_len, n_seg;
    float* seg_state; float* seg_decay;
};

// Segment s of step row r has the slot q_start / seg_len + r + s: slots of different rows never meet, and a step of T
// tokens and n rows needs at most T / seg_len + n + 1 of them.
__device__ __forceinline__ int seg_slot(int q_start, int seg_len, int r, int s) { return q_start / seg_len + r + s; }

template <typename T, int PHASE>
__global__ void __launch_bounds__(SCAN_THREADS)
linear_scan_kernel(const ScanParams p) {
    // blockIdx.x = (row * segments + segment) * tiles + tile of value columns
    const int tiles = (p.dv + SCAN_THREADS / p.DS - 1) / (SCAN_THREADS / p.DS);
    const int rs = blockIdx.x / tiles, tile = blockIdx.x - rs * tiles;
    const int r = rs / p.n_seg, seg = rs - r * p.n_seg, h = blockIdx.y;
    const int slot = p.row_slot[r];
    if (slot < 0) return;
    const int q_start = p.row_q_start[r], q_len = p.row_q_len[r], ctx = p.row_ctx_len[r];
    const int t_begin = PHASE == 0 ? 0 : seg * p.seg_len;
    const int t_end = PHASE == 0 ? q_len : min(q_len, t_begin + p.seg_len);
    if (t_begin >= q_len) return;
    const bool last_seg = t_end == q_len;
    if (PHASE == 1 && last_seg) return;              // nothing follows a sequence's last segment
    const int sslot = PHASE == 0 ? 0 : seg_slot(q_start, p.seg_len, r, seg);
    const int d = p.d, dv = p.dv, DS = p.DS, TC = p.TC;
    const int VT = SCAN_THREADS / DS;
    const int tid = threadIdx.x;
    const int vl = tid / DS, ds = tid - vl * DS;
    const int v = tile * VT + vl;
    const bool v_ok = v < dv;

    extern __shared__ float sm[];
    float* q_s = sm;                    // [TC][d]
    float* b_s = q_s + TC * d;          // [TC][d]
    float* a_s = b_s + TC * d;          // [TC][d] (mode 1)
    float* v_s = a_s + (p.mode ? TC * d : 0);   // [TC][VT]

    const T* proj = static_cast<const T*>(p.proj);
    float* st = p.state + ((size_t)slot * p.H + h) * d * dv;
    // a segment after the first starts from what the chaining left in the slot of the segment before it
    const float* st_in = (PHASE == 3 && seg > 0) ? p.seg_state + ((size_t)(sslot - 1) * p.H + h) * d * dv : st;
    float S[SCAN_RPT];
    float A[PHASE == 1 ? SCAN_RPT : 1];
#pragma unroll
    for (int ii = 0; ii < SCAN_RPT; ++ii) {
        const int i = ii * DS + ds;
        S[ii] = (PHASE != 1 && i < d && v_ok) ? st_in[(size_t)i * dv + v] : 0.f;
        if (PHASE == 1) A[ii] = 1.f;
    }
    const float g = p.mode == 0 ? p.decay[h] : 0.f;
    const int half = p.rot >> 1;

    for (int c0 = t_begin; c0 < t_end; c0 += TC) {
        const int n = min(TC, t_end - c0);
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
                    } else if (i == 0 && h == 0 && tile == 0) {
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
            const int vc = tile * VT + c;
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
                        if (PHASE != 1) o = fmaf(S[ii], qr[i], o);
                    }
                }
            } else {
#pragma unroll
                for (int ii = 0; ii < SCAN_RPT; ++ii) {
                    if (ii * DS >= d) break;
                    const int i = ii * DS + ds;
                    if (i < d) {
                        S[ii] = fmaf(ar[i], S[ii], br[i] * vv);
                        if (PHASE == 1) A[ii] *= ar[i];
                        else o = fmaf(S[ii], qr[i], o);
                    }
                }
            }
            if (PHASE != 1) {
                for (int off = 1; off < DS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
                if (ds == 0 && v_ok) p.out[(size_t)(q_start + c0 + tt) * p.H * dv + h * dv + v] = o;
            }
        }
    }
    if (PHASE == 1) {
        float* u = p.seg_state + ((size_t)sslot * p.H + h) * d * dv;
        float* a = p.seg_decay + ((size_t)sslot * p.H + h) * d;
#pragma unroll
        for (int ii = 0; ii < SCAN_RPT; ++ii) {
            const int i = ii * DS + ds;
            if (i < d && v_ok) u[(size_t)i * dv + v] = S[ii];
            if (i < d && p.mode == 1 && tile == 0 && vl == 0) a[i] = A[ii];
        }
        return;
    }
    if (p.write_state && v_ok && last_seg) {
#pragma unroll
        for (int ii = 0; ii < SCAN_RPT; ++ii) {
            const int i = ii * DS + ds;
            if (i < d) st[(size_t)i * dv + v] = S[ii];
        }
    }
}

// Chains the segments of a sequence: a thread owns one state element of one head and walks the sequence's full segments
// in order, S <- A_s S + U_s, leaving in each segment's slot the state that the next segment starts from.
__global__ void scan_chain_kernel(const ScanParams p) {
    const int r = blockIdx.z, h = blockIdx.y;
    const int slot = p.row_slot[r];
    if (slot < 0) return;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int d = p.d, dv = p.dv;
    if (e >= d * dv) return;
    const int i = e / dv;
    const int q_start = p.row_q_start[r], q_len = p.row_q_len[r];
    const int full = (q_len - 1) / p.seg_len;            // segments that another one follows
    if (full <= 0) return;
    float gl = 1.f;
    if (p.mode == 0) {
        const float g = p.decay[h];
        for (int t = 0; t < p.seg_len; ++t) gl *= g;
    }
    float cur = p.state[((size_t)slot * p.H + h) * d * dv + e];
    const int s0 = seg_slot(q_start, p.seg_len, r, 0);
    for (int s = 0; s < full; ++s) {
        float* u = p.seg_state + ((size_t)(s0 + s) * p.H + h) * d * dv + e;
        const float a = p.mode == 0 ? gl : p.seg_decay[((size_t)(s0 + s) * p.H + h) * d + i];
        cur = fmaf(a, cur, *u);
        *u = cur;
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

constexpr int SCAN_SEG = 64;           // tokens of a segment

template <typename T>
static int scan_launches(const ScanParams& base, int n_rows, int VT, size_t smem, cudaStream_t stream) {
    ScanParams p = base;
    const dim3 block(SCAN_THREADS), one(1, 1, 1);
    const unsigned tiles = (p.dv + VT - 1) / VT;
    if (p.n_seg <= 1) {
        p.phase = 0; p.n_seg = 1;
        return launch("linear_scan", linear_scan_kernel<T, 0>, dim3(tiles * n_rows, p.H, 1), block, smem, stream, one, p);
    }
    const dim3 grid(tiles * n_rows * p.n_seg, p.H, 1);
    p.phase = 1;
    int rc = launch("linear_scan_local", linear_scan_kernel<T, 1>, grid, block, smem, stream, one, p);
    if (rc) return rc;
    rc = launch("linear_scan_chain", scan_chain_kernel, dim3((p.d * p.dv + 255) / 256, p.H, n_rows), dim3(256), 0, stream,
                one, p);
    if (rc) return rc;
    p.phase = 3;
    return launch("linear_scan", linear_scan_kernel<T, 3>, grid, block, smem, stream, one, p);
}

// Tokens of a segment, and the floats of scratch memory that a step of T tokens in n_rows sequences needs to run its
// recurrences in segments (states and gate products of T / segment + n_rows + 1 segment slots).
extern "C" int fd_linear_scan_segment() { return SCAN_SEG; }
extern "C" long long fd_linear_scan_scratch_floats(int T, int n_rows, int H, int d, int dv) {
    return (long long)(T / SCAN_SEG + n_rows + 1) * H * ((long long)d * dv + d);
}

// proj [T, ld] of `dtype` (0 float32, 1 bfloat16) holds q at q_col, k (mode 0) or the gate's pre-activation (mode 1)
// at k_col - H * d columns each - and v at v_col (H * dv columns).  state [slots, H, d, dv] and out [T, H * dv] float.
// mode 0: decay [H], cos_t / sin_t [table_len, rot / 2] (unused when rot == 0), k_scale.  mode 1: lower [H * d].
// max_q_len: the longest portion of the step; with scratch memory (fd_linear_scan_scratch_floats floats for the step's T
// tokens) portions longer than two segments run in segments side by side, otherwise each in one CTA per head and tile.
extern "C" int fd_linear_scan(const void* proj, int ld, int dtype, int q_col, int k_col, int v_col, float* state,
                              float* out, int mode, const float* decay, const float* lower, const float* cos_t,
                              const float* sin_t, int table_len, int rot, float k_scale, const int* row_slot,
                              const int* row_q_start, const int* row_q_len, const int* row_ctx_len, int n_rows, int H,
                              int d, int dv, int write_state, int* status, int T, int max_q_len, float* scratch,
                              long long scratch_floats, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    FD_REQUIRE(H > 0 && d > 0 && dv > 0 && d <= 8 * SCAN_RPT, -2, "linear_scan: %d heads of %d x %d (d at most %d)", H, d,
               dv, 8 * SCAN_RPT);
    FD_REQUIRE(mode == 0 || mode == 1, -2, "linear_scan: unknown mode %d", mode);
    FD_REQUIRE(mode == 1 ? lower != nullptr : decay != nullptr, -2, "linear_scan: the mode's constants are missing");
    FD_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d && (rot == 0 || mode == 1 || (cos_t && sin_t)), -2,
               "linear_scan: %d rotated dimensions of %d", rot, d);
    FD_REQUIRE(H <= 65535, -2, "linear_scan: %d heads", H);
    ScanParams p;
    p.proj = proj; p.ld = ld; p.q_col = q_col; p.k_col = k_col; p.v_col = v_col; p.state = state; p.out = out;
    p.decay = decay; p.lower = lower; p.cos_t = cos_t; p.sin_t = sin_t; p.table_len = table_len;
    p.rot = mode == 0 ? rot : 0; p.k_scale = k_scale;
    p.row_slot = row_slot; p.row_q_start = row_q_start; p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len;
    p.H = H; p.d = d; p.dv = dv; p.mode = mode; p.write_state = write_state; p.status = status;
    p.DS = d <= 4 * SCAN_RPT ? 4 : 8;
    p.TC = d <= 128 ? 16 : 8;
    p.phase = 0; p.seg_len = SCAN_SEG; p.n_seg = 1; p.seg_state = nullptr; p.seg_decay = nullptr;
    if (scratch != nullptr && max_q_len > 2 * SCAN_SEG) {
        const long long slots = T / SCAN_SEG + n_rows + 1;
        FD_REQUIRE(scratch_floats >= fd_linear_scan_scratch_floats(T, n_rows, H, d, dv), -2,
                   "linear_scan: %lld floats of scratch memory for %d tokens in %d sequences", scratch_floats, T, n_rows);
        p.n_seg = (max_q_len + SCAN_SEG - 1) / SCAN_SEG;
        p.seg_state = scratch;
        p.seg_decay = scratch + slots * H * d * dv;
    }
    FD_REQUIRE(n_rows <= 65535 && (long long)n_rows * p.n_seg * ((dv + 15) / 16) < (1ll << 31), -2,
               "linear_scan: %d rows of %d segments", n_rows, p.n_seg);
    const int VT = SCAN_THREADS / p.DS;
    const size_t smem = (size_t)((mode ? 3 : 2) * p.TC * d + p.TC * VT) * sizeof(float);
    if (dtype == 0) return scan_launches<float>(p, n_rows, VT, smem, stream);
    return scan_launches<bf16>(p, n_rows, VT, smem, stream);
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
