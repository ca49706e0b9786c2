// Linear-attention recurrences with a matrix state per head, and the per-head norm that follows them.
//
//   S_t = diag(a_t) S_(t-1) + b_t v_t^T,      o_t = S_t^T q_t          S [d, dv] per sequence and head
//
//  * mode 0 (constant decay): a_t = decay[h] for every channel, b_t = rot(k_t) * k_scale, q_t = rot(q_t); rot turns
//    the first `rot` dimensions of a head at the token's position, dimension i paired with i + rot/2.
//  * mode 1 (forget gate): a_t = f_t = lower + (1 - lower) * sigmoid(z_t) per channel, b_t = 1 - f_t,
//    q_t = silu(zq_t); z and zq are columns of the projection.
//  * mode 2 (decay per key channel): a_t = sigmoid(z_t)^(1/tau) per channel with z a float array of its own (the output
//    of a product of its own), b_t = k_t, q_t = q_t * q_scale.  The power is taken as exp(log sigmoid(z) / tau) with
//    log sigmoid(z) = -log(1 + e^-z) worked out on the side where the exponential cannot overflow.
//
// The state lives in float per cache slot and is carried from step to step; a step's tokens of a sequence are walked in
// order, so the sums of every state element are the same whether a prompt comes whole, in portions or token by token.
// Everything after the projection is float: angles' use, gates, decay, state, output.
//
// A CTA of 128 threads takes one sequence of the step, one head and a tile of value columns.  DS = 4 (d <= 128) or 8
// adjacent lanes share a column and each holds 8, 16 or 32 adjacent rows of it in registers (rows beyond d are
// padding whose q, a and b are zero); the tokens' q, a, b and v are staged in shared memory a chunk at a time by all
// threads, then the chunk is walked token by token: per token a thread reads its rows' q, a and b four at a time, does
// two fused multiply-adds per state element it holds, and the DS lanes add their partial outputs with shuffles.
//
// Long portions (prompts) are cut into segments of `seg_len` tokens that run side by side.  A first launch leaves every
// token's q, a, b and v as floats in the order the recurrence reads them (its CTAs then copy them to shared memory
// with cp.async, a chunk ahead of the one they walk); then three launches:
//  1. every segment but a sequence's last walks its tokens from a zero state and leaves U = its own contribution to
//     the state [d, dv] and, with a forget gate, the product A of its gates per channel (a constant decay's product is
//     decay^seg_len);
//  2. per sequence, head and state element the segments are chained: S_0 = the cached state, S_(s+1) = A_s S_s + U_s;
//  3. every segment walks its tokens again from its S_s and writes the outputs; the last one writes the state back.
// The recurrence itself is unchanged, so nothing is divided by a product of gates that could vanish.
//
//  * low_rank_expand: a narrow vector per token times a matrix [N, R] plus a bias, as floats (the pre-activation of a
//    decay that comes through a narrow projection);
//  * head_norm_gate: y = o / sqrt(mean(o^2) + eps) per token and head (over dv), times an optional weight [dv], times
//    an optional silu(gate) read from a column range of a packed projection, times a constant; written with a row
//    stride and a column offset of its own so that several mixers can fill one buffer.
#include <math.h>

#include "common.cuh"
#include "mma_utils.cuh"

namespace fd {

constexpr int SCAN_THREADS = 128;

struct ScanParams {
    const void* proj; int ld;          // [T, ld]
    int q_col, k_col, v_col;           // first columns of q, of k (mode 0) or the gate's pre-activation (mode 1), of v
    float* state;                      // [slots, H, d, dv]
    float* out;                        // [T, H * dv]
    const float* decay;                // [H] (mode 0)
    const float* lower;                // [H * d] (mode 1)
    const float* gate; int gate_ld;    // [T, gate_ld] from the first of the H * d columns on (mode 2)
    float q_scale, inv_tau;            // (mode 2)
    const float* cos_t; const float* sin_t; int table_len, rot;
    float k_scale;
    const int* row_slot; const int* row_q_start; const int* row_q_len; const int* row_ctx_len;
    int H, d, dv, mode, write_state, DS, TC;
    int* status;
    // segments: phase 0 = the whole portion in one CTA; 1 = a segment from a zero state, leaves U (and A); 3 = a segment
    // from its chained start state, writes outputs.  seg_state [segment slots, H, d, dv], seg_decay [segment slots, H, d].
    int phase, seg_len, n_seg;
    float* seg_state; float* seg_decay;
    float* prep; float* prep_v; int dvp;      // the preparing kernel's q, b (and a) [T, H, NA * CS] and v [T, H, dvp]
};

// Segment s of step row r has the slot q_start / seg_len + r + s: slots of different rows never meet, and a step of T
// tokens and n rows needs at most T / seg_len + n + 1 of them.
__device__ __forceinline__ int seg_slot(int q_start, int seg_len, int r, int s) { return q_start / seg_len + r + s; }

// Shared-memory place of channel i of a token: a thread's NR rows are adjacent (read four at a time), and the DS groups
// of rows are NR + 4 floats apart so that the DS lanes of a column read different banks.
template <int NR> __host__ __device__ constexpr int chan_stride() { return NR == 4 ? 4 : NR + 4; }
template <int NR> __device__ __forceinline__ int chan_at(int i) { return (i / NR) * chan_stride<NR>() + (i % NR); }
constexpr int SCAN_COLS = 4;           // adjacent value columns a thread holds

// q, b (and a) of n tokens from `tok0` on (the first at position pos0), as floats: token tt's q goes to
// dst + tt * tok_stride + chan_at(i), its b CS floats further and its a 2 CS floats further.  A thread's loads of several
// elements are all issued before the first of them is used.
template <typename T, int NR>
__device__ __forceinline__ void stage_tokens(const ScanParams& p, int h, int tok0, int pos0, int n, float* dst,
                                             size_t tok_stride, int DP, int CS, int tid, int n_threads, bool report) {
    const T* proj = static_cast<const T*>(p.proj);
    const int d = p.d, half = p.rot >> 1;
    constexpr int UNR = 4;
    for (int idx0 = tid; idx0 < n * DP; idx0 += n_threads * UNR) {
        float xq[UNR], xk[UNR], yq[UNR], yk[UNR], cc[UNR], ss[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int idx = idx0 + u * n_threads;
            xq[u] = xk[u] = yq[u] = yk[u] = ss[u] = 0.f; cc[u] = 1.f;
            if (idx >= n * DP) continue;
            const int tt = idx / DP, i = idx - tt * DP;
            if (i >= d) continue;
            const size_t row = (size_t)(tok0 + tt) * p.ld;
            xq[u] = to_float(proj[row + p.q_col + h * d + i]);
            xk[u] = to_float(proj[row + p.k_col + h * d + i]);
            if (p.mode == 0 && i < p.rot) {
                const int pos = pos0 + tt;
                if (pos < p.table_len) {
                    const bool first = i < half;
                    const int pi = first ? i : i - half;
                    const int partner = first ? i + half : i - half;
                    cc[u] = p.cos_t[(size_t)pos * half + pi];
                    ss[u] = first ? -p.sin_t[(size_t)pos * half + pi] : p.sin_t[(size_t)pos * half + pi];
                    yq[u] = to_float(proj[row + p.q_col + h * d + partner]);
                    yk[u] = to_float(proj[row + p.k_col + h * d + partner]);
                } else if (i == 0 && report) {
                    set_status(p.status, STATUS_BAD_POSITION);
                }
            } else if (p.mode == 1) {
                cc[u] = p.lower[h * d + i];
            } else if (p.mode == 2) {
                cc[u] = p.gate[(size_t)(tok0 + tt) * p.gate_ld + h * d + i];
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int idx = idx0 + u * n_threads;
            if (idx >= n * DP) continue;
            const int tt = idx / DP, i = idx - tt * DP;
            float* at = dst + tt * tok_stride + chan_at<NR>(i);
            if (i >= d) {
                at[0] = 0.f; at[CS] = 0.f;
                if (p.mode != 0) at[2 * CS] = 0.f;
            } else if (p.mode == 0) {
                at[0] = xq[u] * cc[u] + yq[u] * ss[u];              // first half: x c - y s; second half: x c + y s
                at[CS] = (xk[u] * cc[u] + yk[u] * ss[u]) * p.k_scale;
            } else if (p.mode == 2) {
                const float z = cc[u];
                const float log_sig = z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
                at[0] = xq[u] * p.q_scale;
                at[CS] = xk[u];
                at[2 * CS] = expf(log_sig * p.inv_tau);
            } else {
                const float lo = cc[u];
                const float f = lo + (1.f - lo) / (1.f + expf(-xk[u]));
                at[0] = xq[u] / (1.f + expf(-xq[u]));
                at[CS] = 1.f - f;
                at[2 * CS] = f;
            }
        }
    }
}

constexpr int PREP_TOKENS = 16;        // tokens a CTA of the preparing kernel takes
constexpr int PREP_THREADS = 256;

// Before a step's segments run: q, b (and a) and v of every token as floats in the layout the recurrence reads them
// in, prep [T, H, NA * CS] and prep_v [T, H, dvp], so that its CTAs (several per head, twice over) copy them instead of
// each working them out.  blockIdx.x = (row * segments + segment) * (seg_len / PREP_TOKENS) + part.
template <typename T, int NR>
__global__ void __launch_bounds__(PREP_THREADS)
scan_prepare_kernel(const ScanParams p) {
    const int parts = p.seg_len / PREP_TOKENS;
    const int rs = blockIdx.x / parts, part = blockIdx.x - rs * parts;
    const int r = rs / p.n_seg, seg = rs - r * p.n_seg, h = blockIdx.y;
    if (p.row_slot[r] < 0) return;
    const int q_start = p.row_q_start[r], q_len = p.row_q_len[r], ctx = p.row_ctx_len[r];
    const int t0 = seg * p.seg_len + part * PREP_TOKENS;
    if (t0 >= q_len) return;
    const int n = min(PREP_TOKENS, q_len - t0);
    const int DP = p.DS * NR, CS = p.DS * chan_stride<NR>();
    const size_t TS = (size_t)(p.mode ? 3 : 2) * CS;
    stage_tokens<T, NR>(p, h, q_start + t0, ctx + t0, n, p.prep + ((size_t)(q_start + t0) * p.H + h) * TS, p.H * TS, DP, CS,
                        threadIdx.x, PREP_THREADS, h == 0);
    const T* proj = static_cast<const T*>(p.proj);
    for (int idx = threadIdx.x; idx < n * p.dvp; idx += PREP_THREADS) {
        const int tt = idx / p.dvp, c = idx - tt * p.dvp;
        const size_t tok = q_start + t0 + tt;
        p.prep_v[(tok * p.H + h) * p.dvp + c] = c < p.dv ? to_float(proj[tok * p.ld + p.v_col + h * p.dv + c]) : 0.f;
    }
}

template <typename T, int PHASE, int NR>
__global__ void __launch_bounds__(SCAN_THREADS)
linear_scan_kernel(const ScanParams p) {
    // blockIdx.x = (row * segments + segment) * tiles + tile of value columns
    const int DS = p.DS, TC = p.TC;
    const int VT = SCAN_THREADS / DS * SCAN_COLS;
    const int tiles = (p.dv + VT - 1) / VT;
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
    const int d = p.d, dv = p.dv;
    const int DP = DS * NR;                          // channels with the padding (their q, a and b are zero)
    const int CS = DS * chan_stride<NR>();                    // floats of one of a token's q, b and a in shared memory
    const int TS = (p.mode ? 3 : 2) * CS;            // floats of a token's q, b (and a)
    const int BUF = TC * (TS + VT);                  // floats of a chunk: [TC][TS], then v [TC][VT]
    const int tid = threadIdx.x;
    const int vl = tid / DS, ds = tid - vl * DS;
    const int v0 = tile * VT + vl * SCAN_COLS;       // the thread's columns v0 .. v0 + 3

    extern __shared__ __align__(16) float sm[];     // one chunk (PHASE 0) or two, filled in turn

    float* st = p.state + ((size_t)slot * p.H + h) * d * dv;
    // a segment after the first starts from what the chaining left in the slot of the segment before it
    const float* st_in = (PHASE == 3 && seg > 0) ? p.seg_state + ((size_t)(sslot - 1) * p.H + h) * d * dv : st;
    float S[NR][SCAN_COLS];             // rows ds * NR .. ds * NR + NR - 1 of the thread's columns
    float A[PHASE == 1 ? NR : 1];
#pragma unroll
    for (int ii = 0; ii < NR; ++ii) {
        const int i = ds * NR + ii;
#pragma unroll
        for (int c = 0; c < SCAN_COLS; ++c)
            S[ii][c] = (PHASE != 1 && i < d && v0 + c < dv) ? st_in[(size_t)i * dv + v0 + c] : 0.f;
        if (PHASE == 1) A[ii] = 1.f;
    }
    const float g = p.mode == 0 ? p.decay[h] : 0.f;
    const int my = ds * chan_stride<NR>();

    // segments copy what the preparing kernel left, a chunk ahead of the one that is walked
    auto issue = [&](int c0, int buf) {
        const int n = min(TC, t_end - c0);
        float* dst = sm + buf * BUF;
        const int cpt = TS >> 2, cpv = VT >> 2;      // 16-byte pieces per token
        for (int idx = tid; idx < n * cpt; idx += SCAN_THREADS) {
            const int tt = idx / cpt, c = idx - tt * cpt;
            cp_async16(smem_u32(dst + tt * TS + c * 4), p.prep + ((size_t)(q_start + c0 + tt) * p.H + h) * TS + c * 4, 16);
        }
        for (int idx = tid; idx < n * cpv; idx += SCAN_THREADS) {
            const int tt = idx / cpv, c = idx - tt * cpv;
            const int col = tile * VT + c * 4;
            const bool in = col < p.dvp;
            cp_async16(smem_u32(dst + TC * TS + tt * VT + c * 4),
                       in ? p.prep_v + ((size_t)(q_start + c0 + tt) * p.H + h) * p.dvp + col : p.prep_v, in ? 16 : 0);
        }
        cp_async_commit();
    };
    if (PHASE != 0) issue(t_begin, 0);

    int it = 0;
    for (int c0 = t_begin; c0 < t_end; c0 += TC, ++it) {
        const int n = min(TC, t_end - c0);
        float* buf = sm;
        if (PHASE == 0) {
            __syncthreads();
            stage_tokens<T, NR>(p, h, q_start + c0, ctx + c0, n, sm, TS, DP, CS, tid, SCAN_THREADS, h == 0 && tile == 0);
            const T* proj = static_cast<const T*>(p.proj);
            for (int idx = tid; idx < n * VT; idx += SCAN_THREADS) {
                const int tt = idx / VT, c = idx - tt * VT;
                const int vc = tile * VT + c;
                sm[TC * TS + idx] = vc < dv ? to_float(proj[(size_t)(q_start + c0 + tt) * p.ld + p.v_col + h * dv + vc]) : 0.f;
            }
            __syncthreads();
        } else {
            if (c0 + TC < t_end) {
                issue(c0 + TC, (it + 1) & 1);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            buf = sm + (it & 1) * BUF;
        }
        const float* v_s = buf + TC * TS;
        for (int tt = 0; tt < n; ++tt) {
            const float4 vv = *reinterpret_cast<const float4*>(v_s + tt * VT + vl * SCAN_COLS);
            const float4* qr = reinterpret_cast<const float4*>(buf + tt * TS + my);
            const float4* br = reinterpret_cast<const float4*>(buf + tt * TS + CS + my);
            const float4* ar = reinterpret_cast<const float4*>(buf + tt * TS + 2 * CS + my);
            float o[SCAN_COLS] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < NR / 4; ++j) {
                const float4 b4 = br[j];
                float4 a4 = make_float4(g, g, g, g), q4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (p.mode != 0) a4 = ar[j];
                if (PHASE != 1) q4 = qr[j];
                const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float* Sr = S[4 * j + e];
                    Sr[0] = fmaf(aa[e], Sr[0], bb[e] * vv.x);
                    Sr[1] = fmaf(aa[e], Sr[1], bb[e] * vv.y);
                    Sr[2] = fmaf(aa[e], Sr[2], bb[e] * vv.z);
                    Sr[3] = fmaf(aa[e], Sr[3], bb[e] * vv.w);
                    if (PHASE == 1) {
                        if (p.mode != 0) A[4 * j + e] *= aa[e];
                    } else {
                        o[0] = fmaf(Sr[0], qq[e], o[0]);
                        o[1] = fmaf(Sr[1], qq[e], o[1]);
                        o[2] = fmaf(Sr[2], qq[e], o[2]);
                        o[3] = fmaf(Sr[3], qq[e], o[3]);
                    }
                }
            }
            if (PHASE != 1) {
                for (int off = 1; off < DS; off <<= 1) {
#pragma unroll
                    for (int c = 0; c < SCAN_COLS; ++c) o[c] += __shfl_xor_sync(0xffffffffu, o[c], off);
                }
                if (ds == 0) {
                    float* orow = p.out + (size_t)(q_start + c0 + tt) * p.H * dv + h * dv + v0;
#pragma unroll
                    for (int c = 0; c < SCAN_COLS; ++c)
                        if (v0 + c < dv) orow[c] = o[c];
                }
            }
        }
        if (PHASE != 0) __syncthreads();             // the chunk is through before its place is filled again
    }
    if (PHASE == 1) {
        float* u = p.seg_state + ((size_t)sslot * p.H + h) * d * dv;
        float* a = p.seg_decay + ((size_t)sslot * p.H + h) * d;
#pragma unroll
        for (int ii = 0; ii < NR; ++ii) {
            const int i = ds * NR + ii;
            if (i >= d) continue;
#pragma unroll
            for (int c = 0; c < SCAN_COLS; ++c)
                if (v0 + c < dv) u[(size_t)i * dv + v0 + c] = S[ii][c];
            if (p.mode != 0 && tile == 0 && vl == 0) a[i] = A[ii];
        }
        return;
    }
    if (p.write_state && last_seg) {
#pragma unroll
        for (int ii = 0; ii < NR; ++ii) {
            const int i = ds * NR + ii;
            if (i >= d) continue;
#pragma unroll
            for (int c = 0; c < SCAN_COLS; ++c)
                if (v0 + c < dv) st[(size_t)i * dv + v0 + c] = S[ii][c];
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


// out[t, c] = bias[c] + sum_r w[c, r] * x[t, x_col + r]: a narrow vector per token (R <= EXPAND_MAX_R columns of a wider
// matrix) expanded to N channels, float sums in the order r = 0, 1, ... from the bias on, whatever else the step holds.
// A CTA of two warps takes 64 channels and up to EXPAND_TOK tokens, so that a decode step still spreads over dozens of
// SMs: the tokens' vectors wait in shared memory as floats (every thread reads the same one: a broadcast), and a thread
// streams its own row of w with 16-byte loads, several in flight.
constexpr int EXPAND_MAX_R = 64;
constexpr int EXPAND_TOK = 8;
constexpr int EXPAND_CH = 64;

template <typename T>
__global__ void __launch_bounds__(EXPAND_CH)
low_rank_expand_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ w, const float* __restrict__ bias,
                       float* __restrict__ out, int n_tok, int N, int R) {
    __shared__ __align__(16) float x_s[EXPAND_TOK * EXPAND_MAX_R];
    const int c = blockIdx.x * EXPAND_CH + threadIdx.x, t0 = blockIdx.y * EXPAND_TOK;
    const int nt = min(EXPAND_TOK, n_tok - t0);
    for (int e = threadIdx.x; e < EXPAND_TOK * R; e += EXPAND_CH) {
        const int tt = e / R, r = e - tt * R;
        x_s[e] = tt < nt ? to_float(x[(size_t)(t0 + tt) * ldx + r]) : 0.f;
    }
    __syncthreads();
    if (c >= N) return;
    const float b = bias != nullptr ? bias[c] : 0.f;
    const T* wr = w + (size_t)c * R;
    float acc[EXPAND_TOK];
#pragma unroll
    for (int tt = 0; tt < EXPAND_TOK; ++tt) acc[tt] = b;
    constexpr int VEC = 16 / sizeof(T);
    if (R % VEC == 0 && (uintptr_t)w % 16 == 0) {
#pragma unroll 4
        for (int r0 = 0; r0 < R; r0 += VEC) {
            const uint4 raw = *reinterpret_cast<const uint4*>(wr + r0);
            const T* e = reinterpret_cast<const T*>(&raw);
            float wv[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) wv[j] = to_float(e[j]);
#pragma unroll
            for (int tt = 0; tt < EXPAND_TOK; ++tt) {
                // four values of the token's vector per shared-memory load; the sum still runs over r in order
#pragma unroll
                for (int j4 = 0; j4 < VEC; j4 += 4) {
                    const float4 xv = *reinterpret_cast<const float4*>(x_s + tt * R + r0 + j4);
                    acc[tt] = fmaf(wv[j4], xv.x, acc[tt]);
                    acc[tt] = fmaf(wv[j4 + 1], xv.y, acc[tt]);
                    acc[tt] = fmaf(wv[j4 + 2], xv.z, acc[tt]);
                    acc[tt] = fmaf(wv[j4 + 3], xv.w, acc[tt]);
                }
            }
        }
    } else {
        for (int r = 0; r < R; ++r) {
            const float wv = to_float(wr[r]);
#pragma unroll
            for (int tt = 0; tt < EXPAND_TOK; ++tt) acc[tt] = fmaf(wv, x_s[tt * R + r], acc[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < EXPAND_TOK; ++tt)
        if (tt < nt) out[(size_t)(t0 + tt) * N + c] = acc[tt];
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

constexpr int SCAN_SEG = 64;           // tokens of a segment

template <typename T, int NR>
static int scan_launches(const ScanParams& base, int n_rows, cudaStream_t stream) {
    ScanParams p = base;
    const int VT = SCAN_THREADS / p.DS * SCAN_COLS;
    const dim3 block(SCAN_THREADS), one(1, 1, 1);
    const unsigned tiles = (p.dv + VT - 1) / VT;
    if (p.n_seg <= 1) {
        p.phase = 0; p.n_seg = 1;
        const size_t smem = (size_t)p.TC * ((p.mode ? 3 : 2) * p.DS * chan_stride<NR>() + VT) * sizeof(float);
        return launch("linear_scan", linear_scan_kernel<T, 0, NR>, dim3(tiles * n_rows, p.H, 1), block, smem, stream, one, p);
    }
    p.TC = p.d <= 128 ? 8 : 4;             // two chunks in shared memory, one of them in flight
    const size_t smem = 2 * (size_t)p.TC * ((p.mode ? 3 : 2) * p.DS * chan_stride<NR>() + VT) * sizeof(float);
    int rc = launch("linear_scan_prepare", scan_prepare_kernel<T, NR>,
                    dim3(n_rows * p.n_seg * (p.seg_len / PREP_TOKENS), p.H, 1), dim3(PREP_THREADS), 0, stream, one, p);
    if (rc) return rc;
    const dim3 grid(tiles * n_rows * p.n_seg, p.H, 1);
    p.phase = 1;
    rc = launch("linear_scan_local", linear_scan_kernel<T, 1, NR>, grid, block, smem, stream, one, p);
    if (rc) return rc;
    rc = launch("linear_scan_chain", scan_chain_kernel, dim3((p.d * p.dv + 255) / 256, p.H, n_rows), dim3(256), 0, stream,
                one, p);
    if (rc) return rc;
    p.phase = 3;
    return launch("linear_scan", linear_scan_kernel<T, 3, NR>, grid, block, smem, stream, one, p);
}

// A thread holds NR adjacent rows of four columns; DS lanes share those columns: 8 rows and 16 or 32 lanes for the
// larger heads, 4 rows and as many lanes as cover d for heads up to 64.
static int scan_nr(int d) { return d > 64 ? 8 : 4; }
static int scan_ds(int d) {
    int ds = 4;
    while (ds * scan_nr(d) < d) ds *= 2;
    return ds;
}

template <typename T>
static int scan_by_rows(const ScanParams& p, int n_rows, cudaStream_t stream) {
    if (scan_nr(p.d) == 8) return scan_launches<T, 8>(p, n_rows, stream);
    return scan_launches<T, 4>(p, n_rows, stream);
}

// Tokens of a segment, and the floats of scratch memory that a step of T tokens in n_rows sequences needs to run its
// recurrences in segments: the prepared q, b, a (three places of DS * chan_stride<NR>() floats per token and head) and v, then
// states and gate products of T / segment + n_rows + 1 segment slots.
extern "C" int fd_linear_scan_segment() { return SCAN_SEG; }
static int scan_chan_floats(int d) { return scan_ds(d) * (scan_nr(d) == 4 ? 4 : scan_nr(d) + 4); }
static long long scan_prep_floats(int T, int H, int d, int dv) {
    return (long long)T * H * (3 * scan_chan_floats(d) + (dv + 3) / 4 * 4);
}
extern "C" long long fd_linear_scan_scratch_floats(int T, int n_rows, int H, int d, int dv) {
    return scan_prep_floats(T, H, d, dv) + (long long)(T / SCAN_SEG + n_rows + 1) * H * ((long long)d * dv + d);
}

// proj [T, ld] of `dtype` (0 float32, 1 bfloat16) holds q at q_col, k (mode 0) or the gate's pre-activation (mode 1)
// at k_col - H * d columns each - and v at v_col (H * dv columns).  state [slots, H, d, dv] and out [T, H * dv] float.
// mode 0: decay [H], cos_t / sin_t [table_len, rot / 2] (unused when rot == 0), k_scale.  mode 1: lower [H * d].
// mode 2: gate [T, gate_ld] float (the decay's pre-activation, H * d columns from the pointer on), q_scale, inv_tau.
// max_q_len: the longest portion of the step; with scratch memory (fd_linear_scan_scratch_floats floats for the step's T
// tokens) portions longer than two segments run in segments side by side, otherwise each in one CTA per head and tile.
extern "C" int fd_linear_scan(const void* proj, int ld, int dtype, int q_col, int k_col, int v_col, float* state,
                              float* out, int mode, const float* decay, const float* lower, const float* cos_t,
                              const float* sin_t, int table_len, int rot, float k_scale, const int* row_slot,
                              const int* row_q_start, const int* row_q_len, const int* row_ctx_len, int n_rows, int H,
                              int d, int dv, int write_state, int* status, int T, int max_q_len, float* scratch,
                              long long scratch_floats, const float* gate, int gate_ld, float q_scale, float inv_tau,
                              cudaStream_t stream) {
    if (n_rows == 0) return 0;
    FD_REQUIRE(H > 0 && d > 0 && dv > 0 && d <= 256, -2, "linear_scan: %d heads of %d x %d (d at most 256)", H, d, dv);
    FD_REQUIRE(mode >= 0 && mode <= 2, -2, "linear_scan: unknown mode %d", mode);
    FD_REQUIRE(mode == 1 ? lower != nullptr : (mode == 2 ? gate != nullptr && gate_ld >= H * d : decay != nullptr), -2,
               "linear_scan: the mode's constants are missing");
    FD_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d && (rot == 0 || mode != 0 || (cos_t && sin_t)), -2,
               "linear_scan: %d rotated dimensions of %d", rot, d);
    FD_REQUIRE(H <= 65535, -2, "linear_scan: %d heads", H);
    ScanParams p;
    p.proj = proj; p.ld = ld; p.q_col = q_col; p.k_col = k_col; p.v_col = v_col; p.state = state; p.out = out;
    p.decay = decay; p.lower = lower; p.cos_t = cos_t; p.sin_t = sin_t; p.table_len = table_len;
    p.rot = mode == 0 ? rot : 0; p.k_scale = k_scale;
    p.gate = gate; p.gate_ld = gate_ld; p.q_scale = q_scale; p.inv_tau = inv_tau;
    p.row_slot = row_slot; p.row_q_start = row_q_start; p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len;
    p.H = H; p.d = d; p.dv = dv; p.mode = mode; p.write_state = write_state; p.status = status;
    p.DS = scan_ds(d);
    p.TC = d <= 128 ? 16 : 8;
    p.phase = 0; p.seg_len = SCAN_SEG; p.n_seg = 1; p.seg_state = nullptr; p.seg_decay = nullptr;
    p.prep = nullptr; p.prep_v = nullptr; p.dvp = (dv + 3) / 4 * 4;
    if (scratch != nullptr && max_q_len > 2 * SCAN_SEG) {
        const long long slots = T / SCAN_SEG + n_rows + 1;
        FD_REQUIRE(scratch_floats >= fd_linear_scan_scratch_floats(T, n_rows, H, d, dv), -2,
                   "linear_scan: %lld floats of scratch memory for %d tokens in %d sequences", scratch_floats, T, n_rows);
        p.n_seg = (max_q_len + SCAN_SEG - 1) / SCAN_SEG;
        FD_REQUIRE((uintptr_t)scratch % 16 == 0, -2, "linear_scan: scratch memory must be 16-byte aligned");
        p.prep = scratch;
        p.prep_v = scratch + (long long)T * H * (mode ? 3 : 2) * scan_chan_floats(d);
        p.seg_state = scratch + scan_prep_floats(T, H, d, dv);
        p.seg_decay = p.seg_state + slots * H * d * dv;
    }
    FD_REQUIRE(n_rows <= 65535 && (long long)n_rows * p.n_seg * ((dv + 15) / 16) < (1ll << 31), -2,
               "linear_scan: %d rows of %d segments", n_rows, p.n_seg);
    if (dtype == 0) return scan_by_rows<float>(p, n_rows, stream);
    return scan_by_rows<bf16>(p, n_rows, stream);
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

// x: pointer to the first of the R columns of a matrix [T, ldx] of `dtype` (0 float32, 1 bfloat16); w [N, R] of the same
// type; bias [N] float or null; out [T, N] float.  R at most 64.
extern "C" int fd_low_rank_expand(const void* x, int ldx, const void* w, const float* bias, float* out, int dtype, int T,
                                  int N, int R, cudaStream_t stream) {
    if (T == 0 || N == 0) return 0;
    FD_REQUIRE(R >= 1 && R <= EXPAND_MAX_R && ldx >= R, -2, "low_rank_expand: %d columns of rows of %d (at most %d)", R, ldx, EXPAND_MAX_R);
    const dim3 grid((N + EXPAND_CH - 1) / EXPAND_CH, (T + EXPAND_TOK - 1) / EXPAND_TOK);
    FD_REQUIRE(grid.y <= 65535, -2, "low_rank_expand: %d tokens are too many", T);
    if (dtype == 0)
        return launch("low_rank_expand", low_rank_expand_kernel<float>, grid, dim3(EXPAND_CH), 0, stream, dim3(1, 1, 1),
                      (const float*)x, ldx, (const float*)w, bias, out, T, N, R);
    return launch("low_rank_expand", low_rank_expand_kernel<bf16>, grid, dim3(EXPAND_CH), 0, stream, dim3(1, 1, 1),
                  (const bf16*)x, ldx, (const bf16*)w, bias, out, T, N, R);
}
