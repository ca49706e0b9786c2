// Causal grouped-query attention over the paged KV cache on the CUDA cores,
// for any head size that is a multiple of 8 (up to 256; values may have a
// size of their own), any group size up to 64, any block size, an optional
// sliding window or chunked visibility (keys of the query's own chunk of
// `chunk` positions only, chunks counted from the start of the sequence),
// float or bfloat16 storage.  Options that only this kernel has: scores capped by a
// tanh, a window that also keeps the first positions of the sequence (the key
// tiles between those and the window's start are skipped), a learned term per
// head in the softmax denominator that has no key and no value, and weights that
// are applied to every value head instead of the query head's own (the caller
// mixes the heads' outputs afterwards).  One kernel serves both kinds of step:
//
//  * prompts: a CTA takes QT consecutive query tokens of one sequence and one
//    KV head, i.e. R = QT * G query rows that share the same keys, and walks
//    the keys in tiles of 32;
//  * decode: QT = 1 and the keys of a sequence are cut into n_splits ranges of
//    split_len tokens (flash-decoding); each CTA leaves an unnormalised
//    (max, sum, accumulator) triple per query row in scratch memory and a
//    second kernel merges them.
//
// Tile and split boundaries are fixed in absolute token index, so the order
// of the floating-point sums of a query does not depend on what else is in
// the batch.  Scores, softmax and the value sum are float; bfloat16 is only a
// storage format here.  This is the attention of the true 32-bit path and the
// fallback for head sizes the tensor-core kernels do not take.
#include <math.h>

#include "attention.cuh"

namespace fd {

constexpr int KT = 32;          // keys per tile (= lanes of a warp)
constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int RMAX = 64;        // query rows per CTA
constexpr int RPW = RMAX / ATT_WARPS;   // rows per warp in the score phase
constexpr int RPT_MAX = 16;     // rows per thread in the value phase


// Heads wider than 256 (one cached latent as key and value of many query heads): a CTA takes at most RWIDE query rows,
// which is what its threads' value accumulators and its shared memory hold at those widths.
constexpr int RWIDE = 32;
constexpr int D_MAX = 512;
__host__ __device__ __forceinline__ int q_rows_alloc(int d, int dv) { return d > 256 || dv > 256 ? RWIDE : RMAX; }

template <typename T> struct Pad;            // padding of a key row in shared memory, in elements
template <> struct Pad<float> { static constexpr int v = 4; };
template <> struct Pad<__nv_bfloat16> { static constexpr int v = 4; };

template <typename T> __device__ __forceinline__ float exp_of(float x);
template <> __device__ __forceinline__ float exp_of<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float exp_of<__nv_bfloat16>(float x) { return __expf(x); }

template <typename T> __device__ __forceinline__ void load_chunk4(const T* p, float f[4]);
template <> __device__ __forceinline__ void load_chunk4<float>(const float* p, float f[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_chunk4<__nv_bfloat16>(const __nv_bfloat16* p, float f[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attn_tile_kernel(const AttnParams p) {
    const int b = blockIdx.z;
    // key head and value head; with v_all the CTA applies its weights to all v_rep value heads in turn (VR of them)
    const int VR = p.v_all ? p.v_rep : 1;
    const int kvh = p.v_all ? blockIdx.y : blockIdx.y / p.v_rep;
    const int vh = p.v_all ? 0 : (p.v_rep > 1 ? blockIdx.y - kvh * p.v_rep : kvh);
    const int tile = blockIdx.x / p.n_splits, split = blockIdx.x - tile * p.n_splits;
    const int slot = p.row_slot[b];
    if (slot < 0) return;
    const int q_len = p.row_q_len[b];
    if (tile * p.QT >= q_len) return;
    const int ctx = p.row_ctx_len[b];
    const int tok0 = p.row_q_start[b] + tile * p.QT;       // first query token of this CTA
    const int nq = min(p.QT, q_len - tile * p.QT);
    const int G = p.G, d = p.d, dv = p.dv;
    const int R = nq * G;
    const int p_first = ctx + tile * p.QT;                  // position of the first query token
    int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    if (p.chunk > 0) lo = max(lo, (p_first / p.chunk) * p.chunk);   // the earliest chunk start among the tile's queries
    int hi = p_first + nq;                                   // keys 0 .. last query position
    // kept first positions that lie before the window's start: keys [s_lo, kf) are visited too, the tiles between skipped
    int kf = (p.window > 0 && p.keep_first > 0) ? min(p.keep_first, lo) : 0;
    int s_lo = 0;
    if (p.n_splits > 1) {
        s_lo = split * p.split_len;
        lo = max(lo, s_lo);
        hi = min(hi, (split + 1) * p.split_len);
        kf = min(kf, hi);
    }
    if (kf <= s_lo) kf = 0;
    const int t_begin = kf > 0 ? (s_lo / KT) * KT : (lo / KT) * KT;
    const int kf_end = ((kf + KT - 1) / KT) * KT, lo_tile = (lo / KT) * KT;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int KPAD = Pad<T>::v;
    const int kstride = d + KPAD;
    float* q_s = reinterpret_cast<float*>(smem_raw);               // [RMAX][d] ([RWIDE][d] for heads wider than 256)
    float* p_s = q_s + q_rows_alloc(d, dv) * d;                       // [RMAX][KT]
    float* alpha_s = p_s + RMAX * KT;                                 // [RMAX]
    float* l_s = alpha_s + RMAX;                                      // [RMAX]
    T* v_s = reinterpret_cast<T*>(l_s + RMAX);                        // [VR][KT][dv]
    T* k_s = v_s + VR * KT * dv;                                      // [KT][d + KPAD]

    __shared__ int row_s[KT];                    // per token of the tile: its row in the pools, -1 outside [lo, hi)
    __shared__ int vrow_s[KT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* qg = static_cast<const T*>(p.q);
    const T* kp = static_cast<const T*>(p.k_pool);
    const T* vp = static_cast<const T*>(p.v_pool);

    // queries of this CTA, scaled, as float
    for (int e = tid; e < R * d; e += ATT_THREADS) {
        const int r = e / d, j = e - r * d;
        const int qi = r / G, g = r - qi * G;
        q_s[e] = to_float(qg[((size_t)(tok0 + qi) * p.n_q + kvh * G + g) * d + j]) * p.scale;
    }

    float m_run[RPW], l_run[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

    // value phase mapping: a thread owns 4 consecutive dims of several rows
    const int DC = d >> 2;
    const int DCV = dv >> 2;
    const int RG = ATT_THREADS / DCV;
    const int dc = tid % DCV, rg = tid / DCV;
    const bool pv_active = rg < RG;
    float acc[RPT_MAX][4];
#pragma unroll
    for (int i = 0; i < RPT_MAX; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

    constexpr int EPC = 16 / sizeof(T);          // elements per 16-byte chunk
    const int cpr = d / EPC;                      // chunks per key row
    const int cprv = dv / EPC;                    // chunks per value row
    const int bs = p.block_size;

    for (int t0 = t_begin; t0 < hi; t0 += KT) {
        if (t0 >= kf_end && t0 < lo_tile) t0 = lo_tile;          // nothing visible between the kept keys and the window
        if (t0 >= hi) break;
        __syncthreads();   // previous tile consumed (and q_s written, first time round)
        // stage keys and values of this tile; tokens outside [lo, hi) read as zero.  The tile's block numbers are looked
        // up once per token, then every thread has several independent 16-byte loads in flight (one lookup and one
        // load at a time, each waiting for the one before, made a decode step at wide heads four times as long)
        if (tid < KT) {
            const int t = t0 + tid;
            int base = -1;
            int vbase = -1;
            if ((t >= lo || (t < kf && t >= s_lo)) && t < hi) {
                const int blk = p.block_table[(size_t)slot * p.max_blocks + t / bs];
                if (blk < 0 || blk >= p.num_blocks) set_status(p.status, STATUS_BAD_BLOCK);
                else {
                    base = (blk * p.n_kv + kvh) * bs + (t % bs);          // the token's row in the key pool
                    vbase = (blk * p.n_kv + vh) * bs + (t % bs);          // and in the value pool
                }
            }
            row_s[tid] = base;
            vrow_s[tid] = vbase;
        }
        __syncthreads();
        {
            constexpr int UNR = 4;
            const int per_tok = cpr + cprv * VR, total = KT * per_tok;
            for (int c0 = tid; c0 < total; c0 += ATT_THREADS * UNR) {
                uint4 x4[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int c = c0 + u * ATT_THREADS;
                    x4[u] = make_uint4(0, 0, 0, 0);
                    if (c < total) {
                        const int tt = c / per_tok, cc = c - tt * per_tok;
                        const int base = row_s[tt];
                        if (base >= 0) {
                            const int cv = cc - cpr, j = cv >= 0 ? cv / cprv : 0;       // value head j's row: j * bs rows on
                            x4[u] = cc >= cpr ? *reinterpret_cast<const uint4*>(vp + ((size_t)vrow_s[tt] + (size_t)j * bs) * dv +
                                                                                (cv - j * cprv) * EPC)
                                              : *reinterpret_cast<const uint4*>(kp + (size_t)base * d + cc * EPC);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int c = c0 + u * ATT_THREADS;
                    if (c < total) {
                        const int tt = c / per_tok, cc = c - tt * per_tok;
                        if (cc >= cpr) {
                            const int cv = cc - cpr, j = cv / cprv;
                            *reinterpret_cast<uint4*>(v_s + (j * KT + tt) * dv + (cv - j * cprv) * EPC) = x4[u];
                        } else {
                            uint2* kd = reinterpret_cast<uint2*>(k_s + tt * kstride + cc * EPC);
                            kd[0] = make_uint2(x4[u].x, x4[u].y);
                            kd[1] = make_uint2(x4[u].z, x4[u].w);
                        }
                    }
                }
            }
        }
        __syncthreads();

        // scores: warp `warp` owns rows warp, warp + 8, ...; a lane is a key
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.f;
        const T* krow = k_s + lane * kstride;
        for (int c = 0; c < DC; ++c) {
            float kf[4];
            load_chunk4<T>(krow + c * 4, kf);
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const int r = warp + i * ATT_WARPS;
                if (r >= R) break;          // rows grow with i: nothing of a decode step's few rows is left (the unrolled
                                            // loops' skipped iterations were most of this kernel's instructions there)
                const float4 qv = *reinterpret_cast<const float4*>(q_s + r * d + c * 4);
                s[i] = fmaf(qv.x, kf[0], s[i]);
                s[i] = fmaf(qv.y, kf[1], s[i]);
                s[i] = fmaf(qv.z, kf[2], s[i]);
                s[i] = fmaf(qv.w, kf[3], s[i]);
            }
        }
        // online softmax, one row per warp at a time
        const int t = t0 + lane;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp + i * ATT_WARPS;
            if (r >= R) break;
            {
                const int qpos = p_first + r / G;
                const bool valid = (t >= lo || (t < kf && t >= s_lo)) && t < hi && t <= qpos &&
                                   (p.window <= 0 || qpos - t < p.window || t < p.keep_first) &&
                                   (p.chunk <= 0 || t >= (qpos / p.chunk) * p.chunk);
                float sc = s[i];
                if (p.softcap > 0.f) sc = p.softcap * tanhf(sc / p.softcap);
                const float sv = valid ? sc : -INFINITY;
                const float m_new = fmaxf(m_run[i], warp_max(sv));
                float pr = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {
                    pr = valid ? exp_of<T>(sv - m_new) : 0.f;
                    alpha = exp_of<T>(m_run[i] - m_new);
                }
                l_run[i] = l_run[i] * alpha + warp_sum(pr);
                m_run[i] = m_new;
                p_s[r * KT + lane] = pr;
                if (lane == 0) alpha_s[r] = alpha;
            }
        }
        __syncthreads();

        // values: acc[r][dims] = acc * alpha + sum_t p[r][t] * v[t][dims]
        if (pv_active && VR > 1) {
            // rows R * j + r stand for query row r on value head j: all threads have work although R is small
#pragma unroll
            for (int i = 0; i < RPT_MAX; ++i) {
                const int rv = rg + i * RG;
                if (rv >= R * VR) break;
                const int j = rv / R, r = rv - j * R;
                const float a = alpha_s[r];
                acc[i][0] *= a; acc[i][1] *= a; acc[i][2] *= a; acc[i][3] *= a;
                const T* vj = v_s + (size_t)j * KT * dv + dc * 4;
                for (int tt = 0; tt < KT; ++tt) {
                    float vf[4];
                    load_chunk4<T>(vj + tt * dv, vf);
                    const float pr = p_s[r * KT + tt];
                    acc[i][0] = fmaf(pr, vf[0], acc[i][0]);
                    acc[i][1] = fmaf(pr, vf[1], acc[i][1]);
                    acc[i][2] = fmaf(pr, vf[2], acc[i][2]);
                    acc[i][3] = fmaf(pr, vf[3], acc[i][3]);
                }
            }
        } else if (pv_active) {
#pragma unroll
            for (int i = 0; i < RPT_MAX; ++i) {
                const int r = rg + i * RG;
                if (r >= R) break;
                const float a = alpha_s[r];
                acc[i][0] *= a; acc[i][1] *= a; acc[i][2] *= a; acc[i][3] *= a;
            }
            for (int tt = 0; tt < KT; ++tt) {
                float vf[4];
                load_chunk4<T>(v_s + tt * dv + dc * 4, vf);
#pragma unroll
                for (int i = 0; i < RPT_MAX; ++i) {
                    const int r = rg + i * RG;
                    if (r >= R) break;
                    const float pr = p_s[r * KT + tt];
                    acc[i][0] = fmaf(pr, vf[0], acc[i][0]);
                    acc[i][1] = fmaf(pr, vf[1], acc[i][1]);
                    acc[i][2] = fmaf(pr, vf[2], acc[i][2]);
                    acc[i][3] = fmaf(pr, vf[3], acc[i][3]);
                }
            }
        }
    }

    // hand the row sums (and maxima, when splitting) to the value threads
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp + i * ATT_WARPS;
            if (r < R) { l_s[r] = l_run[i]; alpha_s[r] = m_run[i]; }
        }
    }
    __syncthreads();
    if (!pv_active) return;
    T* og = static_cast<T*>(p.out);
#pragma unroll
    for (int i = 0; i < RPT_MAX; ++i) {
        const int rv = rg + i * RG;
        if (rv >= R * VR) continue;
        const int jv = rv / R, r = rv - jv * R;
        const int qi = r / G, g = r - qi * G;
        const int head = kvh * G + g;
        size_t row = (size_t)(tok0 + qi) * p.n_q + head;
        if (p.v_rep > 1) row = row * p.v_rep + vh + jv;
        if (p.n_splits > 1) {
            const size_t pi = row * p.n_splits + split;
            if (dc == 0) { p.part_m[pi] = alpha_s[r]; p.part_l[pi] = l_s[r]; }
            *reinterpret_cast<float4*>(p.part_acc + pi * dv + dc * 4) =
                make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        } else {
            float l = l_s[r], f = 1.f;
            if (p.sink != nullptr) {                 // one more term in the denominator: exp(sink), no key, no value
                const float sk = p.sink[head], m = alpha_s[r];
                const float m2 = fmaxf(m, sk);
                f = m == -INFINITY ? 0.f : expf(m - m2);
                l = l * f + expf(sk - m2);
            }
            const float inv = l > 0.f ? f / l : 0.f;
            if (p.out_f32) {
                *reinterpret_cast<float4*>(static_cast<float*>(p.out) + row * dv + dc * 4) =
                    make_float4(acc[i][0] * inv, acc[i][1] * inv, acc[i][2] * inv, acc[i][3] * inv);
            } else {
                T* o = og + row * dv + dc * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = from_float<T>(acc[i][j] * inv);
            }
        }
    }
}

// Merge the per-split triples of every (token, query head): m = max m_s,
// l = sum l_s e^(m_s - m), out = sum acc_s e^(m_s - m) / l.  Splits that saw
// no key (l_s == 0) are skipped; a padding row gives zeros.  The weights
// e^(m_s - m) / l are computed once per (token, head) into shared memory; then
// a thread owns one output dim and sums over the splits with independent loads.
constexpr int COMBINE_MAX_SPLITS = 512;

template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                    const float* __restrict__ part_acc, T* __restrict__ out,
                                    const int* __restrict__ tok_row, const int* __restrict__ row_slot,
                                    int n_q, int d, int n_splits, const float* __restrict__ sink, int v_rep,
                                    int out_f32) {
    __shared__ float w_s[COMBINE_MAX_SPLITS];
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int tok = blockIdx.y, h = blockIdx.x;
    const size_t row = (size_t)tok * n_q + h;
    T* o = out + row * d;
    float* of = reinterpret_cast<float*>(out) + row * d;       // the same row when the output is float whatever T is
    if (row_slot[tok_row[tok]] < 0) {
        for (int j = threadIdx.x; j < d; j += blockDim.x) { if (out_f32) of[j] = 0.f; else o[j] = from_float<T>(0.f); }
        return;
    }
    const float* pm = part_m + row * n_splits;
    const float* pl = part_l + row * n_splits;
    // block-wide max of m over the splits that saw a key
    float m = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x)
        if (pl[s] > 0.f) m = fmaxf(m, pm[s]);
    m = warp_max(m);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < nwarps; ++w) m = fmaxf(m, red[w]);
    const float sk = sink != nullptr ? sink[h / v_rep] : -INFINITY;     // the denominator's keyless term
    m = fmaxf(m, sk);
    __syncthreads();
    // weights and their sum, in split order within a thread; the block sum order is fixed too
    float lsum = 0.f;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {
        const float ls = pl[s];
        const float w = ls > 0.f ? expf(pm[s] - m) : 0.f;
        w_s[s] = w;
        lsum += ls * w;
    }
    float l = block_sum(lsum, red);
    if (sink != nullptr) l += expf(sk - m);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float* pa = part_acc + row * n_splits * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float a = 0.f;
        int s = 0;
        for (; s + 4 <= n_splits; s += 4) {
            const float a0 = pa[(size_t)(s + 0) * d + j], a1 = pa[(size_t)(s + 1) * d + j];
            const float a2 = pa[(size_t)(s + 2) * d + j], a3 = pa[(size_t)(s + 3) * d + j];
            a = fmaf(a0, w_s[s], a); a = fmaf(a1, w_s[s + 1], a);
            a = fmaf(a2, w_s[s + 2], a); a = fmaf(a3, w_s[s + 3], a);
        }
        for (; s < n_splits; ++s) a = fmaf(pa[(size_t)s * d + j], w_s[s], a);
        if (out_f32) of[j] = a * inv; else o[j] = from_float<T>(a * inv);
    }
}

template <typename T>
static size_t attn_smem_bytes(int d, int dv, int vr = 1) {
    return (size_t)(q_rows_alloc(d, dv) * d + RMAX * KT + 2 * RMAX) * sizeof(float) +
           (size_t)(vr * KT * dv + KT * (d + Pad<T>::v)) * sizeof(T);
}

template <typename T>
static int launch_attn(const AttnParams& p0, int n_rows, int max_q_len, cudaStream_t stream) {
    AttnParams p = p0;
    // few query rows and repeated value heads: one CTA per key head takes all value heads, if their tiles fit
    p.v_all = p.v_rep > 1 && p.QT * p.G * p.v_rep <= RMAX && p.d <= 256 && p.dv <= 256 &&
              attn_smem_bytes<T>(p.d, p.dv, p.v_rep) <= 160 * 1024;
    const size_t smem = attn_smem_bytes<T>(p.d, p.dv, p.v_all ? p.v_rep : 1);
    auto k = attn_tile_kernel<T>;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-3, "attention: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    const int q_tiles = (max_q_len + p.QT - 1) / p.QT;
    dim3 grid(q_tiles * p.n_splits, p.v_all ? p.n_kv : p.n_kv * p.v_rep, n_rows);
    k<<<grid, ATT_THREADS, smem, stream>>>(p);
    return check_launch("attention");
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// Largest number of query tokens a CTA takes for a group size (0: unsupported).
extern "C" int fd_attn_simt_qt(int G) { return G >= 1 && G <= RMAX ? (RMAX / G > 16 ? 16 : RMAX / G) : 0; }

// Query heads per group the tensor-core decode kernel works on when a key/value head serves G of them: G itself up to
// 16, else G's largest divisor up to 8 (the kernel's faster form), else up to 16; 0: the kernel does not take the sizes.
extern "C" int fd_attn_decode_group(int G, int d, int dv) {
    if (d != dv || (d != 64 && d != 128) || G < 1) return 0;
    if (G <= 16) return G;
    for (int g = 8; g >= 4; --g) if (G % g == 0) return g;
    for (int g = 16; g >= 2; --g) if (G % g == 0) return g;
    return 0;
}

// Floats of scratch the split form needs: part_acc [T, n_q, n_splits, d] (d: the size of a value head), then part_m
// and part_l [T, n_q, n_splits].
extern "C" long long fd_attn_scratch_floats(int T, int n_q, int d, int n_splits) {
    return (long long)T * n_q * n_splits * (d + 2);
}

// dtype: 0 = float32, 1 = bfloat16 (queries, cache and output alike).
// n_splits == 1 writes `out` directly; otherwise `scratch` must hold
// fd_attn_scratch_floats(T, ...) floats and the merge kernel runs after.
// use_mma != 0: decode steps (max_q_len == 1) in bfloat16 go to the
// tensor-core kernel when it takes the head size and group size.
static int attention_impl(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                          const int* block_table, int max_blocks, int num_blocks, int block_size,
                          const int* tok_row, const int* row_slot, const int* row_q_start,
                          const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                          int max_q_len, int n_q, int n_kv, int d, float scale, int window, int dv, int chunk,
                          int n_splits, int split_len, float* scratch, int* counters, int* status, int use_mma,
                          cudaStream_t stream, const void* prefetch = nullptr, unsigned long long prefetch_bytes = 0,
                          float softcap = 0.f, int keep_first = 0, const float* sink = nullptr, int v_rep = 1,
                          int out_f32 = 0, int ext_mma = 0) {
    if (n_rows == 0 || T == 0) return 0;
    FD_REQUIRE(softcap >= 0.f && keep_first >= 0 && v_rep >= 1 && (v_rep == 1 || v_rep == n_kv), -2,
               "attention: soft cap %g, %d kept first keys, weights applied to %d value heads of %d", softcap, keep_first,
               v_rep, n_kv);
    const bool ext = softcap > 0.f || (keep_first > 0 && window > 0) || sink != nullptr || v_rep > 1 || out_f32;
    if (ext) use_mma = 0;
    // of the options the tensor-core decode kernel has the keyless term: a decode step that asks for nothing else runs there
    const bool sink_only = sink != nullptr && !(softcap > 0.f) && !(keep_first > 0 && window > 0) && v_rep == 1 && !out_f32;
    const bool decode_mma = (use_mma != 0 || (sink_only && ext_mma != 0)) && dtype == 1 && max_q_len == 1 && dv == d;
    FD_REQUIRE(n_kv > 0 && n_q % n_kv == 0, -2, "attention: %d query heads are not a multiple of %d KV heads", n_q, n_kv);
    const int G = n_q / n_kv;
    FD_REQUIRE(d % 8 == 0 && d >= 8 && d <= D_MAX, -2, "attention: head size %d must be a multiple of 8 in [8, %d]", d, D_MAX);
    FD_REQUIRE(dv % 8 == 0 && dv >= 8 && dv <= D_MAX, -2, "attention: value head size %d must be a multiple of 8 in [8, %d]", dv, D_MAX);
    FD_REQUIRE((d <= 256 && dv <= 256) || G <= RWIDE, -2, "attention: heads wider than 256 take groups of up to %d query heads, got %d", RWIDE, G);
    FD_REQUIRE(chunk >= 0 && window >= 0, -2, "attention: chunk %d and window %d must not be negative", chunk, window);
    FD_REQUIRE(G <= RMAX, -2, "attention: group size %d exceeds %d", G, RMAX);
    FD_REQUIRE(block_size > 0, -2, "attention: block size %d", block_size);
    FD_REQUIRE(n_splits >= 1 && n_splits <= COMBINE_MAX_SPLITS, -2, "attention: n_splits=%d (1..%d)", n_splits, COMBINE_MAX_SPLITS);
    FD_REQUIRE(n_splits == 1 || (split_len > 0 && split_len % KT == 0), -2,
               "attention: split length %d must be a positive multiple of %d", split_len, KT);
    FD_REQUIRE(n_splits == 1 || scratch != nullptr, -2, "attention: split form needs scratch memory");
    FD_REQUIRE((uintptr_t)scratch % 16 == 0 && (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0 &&
               (uintptr_t)q % 16 == 0, -2,
               "attention: queries, cache pools and scratch memory must be 16-byte aligned");
    FD_REQUIRE(n_splits == 1 || T <= 65535, -2, "attention: the split form takes at most 65535 tokens, got %d", T);
    FD_REQUIRE(n_rows <= 65535 && n_kv <= 65535, -2, "attention: batch of %d rows too large", n_rows);

    AttnParams p;
    p.pf_ptr = (const unsigned char*)prefetch; p.pf_bytes = prefetch ? prefetch_bytes : 0;
    p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.out = out;
    const size_t n_part = (size_t)T * n_q * v_rep * n_splits;
    // accumulators first: they are stored as float4 and must stay 16-byte aligned
    p.part_acc = scratch;
    p.part_m = scratch ? scratch + n_part * dv : nullptr;
    p.part_l = scratch ? scratch + n_part * dv + n_part : nullptr;
    p.block_table = block_table; p.row_slot = row_slot; p.row_q_start = row_q_start;
    p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len; p.status = status;
    p.counters = nullptr;
    p.max_blocks = max_blocks; p.num_blocks = num_blocks; p.block_size = block_size;
    p.n_q = n_q; p.n_kv = n_kv; p.G = G; p.d = d; p.dv = dv; p.chunk = chunk;
    p.n_kv_pool = n_kv; p.kv_div = 1;
    p.softcap = softcap; p.keep_first = keep_first; p.sink = sink; p.v_rep = v_rep; p.out_f32 = out_f32; p.v_all = 0;
    if (dv != d) use_mma = 0;          // the tensor-core kernels keep keys and values of one size
    int qt = fd_attn_simt_qt(G);
    if ((d > 256 || dv > 256) && qt > RWIDE / G) qt = RWIDE / G;
    if (qt > max_q_len) qt = max_q_len;
    p.QT = qt; p.n_splits = n_splits; p.split_len = split_len; p.window = window; p.scale = scale;

    int rc = 1;
    if (decode_mma) {
        AttnParams pd = p;
        const int cut = fd_attn_decode_group(G, d, dv);     // a large group as several smaller ones on the same pool head
        if (cut > 0 && cut < G) { pd.G = cut; pd.kv_div = G / cut; pd.n_kv = n_kv * (G / cut); }
        pd.counters = n_splits > 1 ? counters : nullptr;    // given: the kernel merges its own splits
        rc = pd.n_kv <= 65535 ? launch_attn_decode_mma(pd, n_rows, stream) : 1;
        if (rc == 0 && pd.counters != nullptr) return 0;
    }
    else if (use_mma && dtype == 1) {
        rc = use_mma == 2 ? 1 : launch_attn_prefill_tcgen05(p, n_rows, T, max_q_len, stream);
        if (rc == 1) rc = launch_attn_prefill_mma(p, n_rows, max_q_len, stream);
    }
    if (ext && ext_mma && dtype == 1 && max_q_len > 1) {
        // of the options the tcgen05 prompt kernel has the keyless term too (head size 128)
        if (sink_only && dv == d) rc = launch_attn_prefill_tcgen05(p, n_rows, T, max_q_len, stream);
        if (rc == 1) rc = launch_attn_prefill_mma_ext(p, n_rows, max_q_len, stream);
    }
    if (rc == 1)
        rc = dtype == 0 ? launch_attn<float>(p, n_rows, max_q_len, stream)
                        : launch_attn<bf16>(p, n_rows, max_q_len, stream);
    if (rc != 0 || n_splits == 1) return rc;
    dim3 grid(n_q * v_rep, T);
    if (dtype == 0)
        return launch("attention_combine", attn_combine_kernel<float>, grid, dim3(128), 0, stream, dim3(1, 1, 1),
                      (const float*)p.part_m, (const float*)p.part_l, (const float*)p.part_acc, (float*)out, tok_row,
                      row_slot, n_q * v_rep, dv, n_splits, sink, v_rep, out_f32);
    return launch("attention_combine", attn_combine_kernel<bf16>, grid, dim3(128), 0, stream, dim3(1, 1, 1),
                  (const float*)p.part_m, (const float*)p.part_l, (const float*)p.part_acc, (bf16*)out, tok_row,
                  row_slot, n_q * v_rep, dv, n_splits, sink, v_rep, out_f32);
}

// out[t, h, :] = scale * sum_g mix[h, g] * o[t, g, vh(h), :] with vh(h) = h / (n_q / n_kv): every head takes the other
// heads' weights on the values of its own key/value head.  o [T, n_q, n_kv, dv] float; out rows of ld_out elements.
template <typename T>
__global__ void attn_head_mix_kernel(const float* __restrict__ o, const float* __restrict__ mix, T* __restrict__ out,
                                     int ld_out, int n_q, int n_kv, int dv, float scale) {
    const int t = blockIdx.y, h = blockIdx.x;
    const int vh = h / (n_q / n_kv);
    const float* ot = o + (size_t)t * n_q * n_kv * dv;
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
        float a = 0.f;
        for (int g = 0; g < n_q; ++g) a = fmaf(mix[h * n_q + g], ot[((size_t)g * n_kv + vh) * dv + j], a);
        out[(size_t)t * ld_out + h * dv + j] = from_float<T>(a * scale);
    }
}

// The same with a CTA per token and key/value head: the other heads' outputs on that value head (n_q x dv floats) and the
// group's rows of the mixing matrix are brought to shared memory once, with all loads in flight together, and the G heads
// of the group are summed from there.  Same order of additions as the kernel above.
template <typename T>
__global__ void attn_head_mix_staged_kernel(const float* __restrict__ o, const float* __restrict__ mix, T* __restrict__ out,
                                            int ld_out, int n_q, int n_kv, int dv, float scale) {
    extern __shared__ __align__(16) float mix_sm[];
    const int t = blockIdx.y, vh = blockIdx.x;
    const int G = n_q / n_kv;
    float* o_s = mix_sm;                    // [n_q][dv]
    float* m_s = o_s + n_q * dv;            // [G][n_q]
    const float* ot = o + (size_t)t * n_q * n_kv * dv;
    const int dv4 = dv >> 2;
    for (int e = threadIdx.x; e < n_q * dv4; e += blockDim.x) {
        const int g = e / dv4, c = e - g * dv4;
        reinterpret_cast<float4*>(o_s)[e] = *reinterpret_cast<const float4*>(ot + ((size_t)g * n_kv + vh) * dv + c * 4);
    }
    for (int e = threadIdx.x; e < G * n_q; e += blockDim.x) m_s[e] = mix[(size_t)vh * G * n_q + e];
    __syncthreads();
    for (int e = threadIdx.x; e < G * dv; e += blockDim.x) {
        const int gi = e / dv, j = e - gi * dv;
        float a = 0.f;
        for (int g = 0; g < n_q; ++g) a = fmaf(m_s[gi * n_q + g], o_s[g * dv + j], a);
        out[(size_t)t * ld_out + (vh * G + gi) * dv + j] = from_float<T>(a * scale);
    }
}

// The CUDA-core kernel for every case.
extern "C" int fd_attention_simt(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                 const int* block_table, int max_blocks, int num_blocks, int block_size,
                                 const int* tok_row, const int* row_slot, const int* row_q_start,
                                 const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                                 int max_q_len, int n_q, int n_kv, int d, float scale, int window, int dv, int chunk,
                                 int n_splits, int split_len, float* scratch, int* status,
                                 cudaStream_t stream) {
    return attention_impl(q, k_pool, v_pool, out, dtype, block_table, max_blocks, num_blocks, block_size, tok_row,
                          row_slot, row_q_start, row_q_len, row_ctx_len, n_rows, T, max_q_len, n_q, n_kv, d, scale,
                          window, dv, chunk, n_splits, split_len, scratch, nullptr, status, 0, stream);
}

// The fastest kernel that takes the sizes: tensor cores where possible.  `counters`
// (optional): n_rows * n_kv ints, all zero, which the decode kernel uses to let the last CTA of
// a (sequence, KV head) merge the splits itself (it leaves them zero again); without them the
// separate merge kernel runs.  prefetch / prefetch_bytes (optional, 16-byte aligned): memory that a
// later kernel streams, which the tensor-core decode kernel asks L2 for when its own reads are
// through (the other kernels ignore it).
extern "C" int fd_attention(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                            const int* block_table, int max_blocks, int num_blocks, int block_size,
                            const int* tok_row, const int* row_slot, const int* row_q_start,
                            const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                            int max_q_len, int n_q, int n_kv, int d, float scale, int window, int dv, int chunk,
                            int n_splits, int split_len, float* scratch, int* counters, int* status,
                            const void* prefetch, unsigned long long prefetch_bytes, cudaStream_t stream) {
    FD_REQUIRE((uintptr_t)prefetch % 16 == 0, -2, "attention: the memory to prefetch must be 16-byte aligned");
    return attention_impl(q, k_pool, v_pool, out, dtype, block_table, max_blocks, num_blocks, block_size, tok_row,
                          row_slot, row_q_start, row_q_len, row_ctx_len, n_rows, T, max_q_len, n_q, n_kv, d, scale,
                          window, dv, chunk, n_splits, split_len, scratch, counters, status, 1, stream, prefetch, prefetch_bytes);
}

// The same without the tcgen05 kernel: prompts go to the mma.sync kernel (head sizes other than 128 always
// do; this entry lets tests and measurements reach it at 128 too).
extern "C" int fd_attention_mma_sync(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                     const int* block_table, int max_blocks, int num_blocks, int block_size,
                                     const int* tok_row, const int* row_slot, const int* row_q_start,
                                     const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                                     int max_q_len, int n_q, int n_kv, int d, float scale, int window, int dv, int chunk,
                                     int n_splits, int split_len, float* scratch, int* counters, int* status,
                                     cudaStream_t stream) {
    return attention_impl(q, k_pool, v_pool, out, dtype, block_table, max_blocks, num_blocks, block_size, tok_row,
                          row_slot, row_q_start, row_q_len, row_ctx_len, n_rows, T, max_q_len, n_q, n_kv, d, scale,
                          window, dv, chunk, n_splits, split_len, scratch, counters, status, 2, stream);
}

// Attention with more options (on the CUDA cores; prompts in bfloat16 with heads of 64 or 128 on the tensor cores when
// use_mma is set): softcap > 0 caps the scaled scores by a tanh; keep_first: with a window, the
// first so many positions stay visible; sink [n_q] (or null): a keyless term exp(sink[h]) in head h's denominator;
// v_rep == n_kv: every query head's weights are applied to all value heads and out is [T, n_q, n_kv, dv] (scratch for
// the split form: fd_attn_scratch_floats(T, n_q * n_kv, dv, n_splits)); out_f32: out is float.  Decode steps in bfloat16
// whose only option is the keyless term run on the tensor-core decode kernel when use_mma is set and it takes the sizes
// (counters: as for fd_attention, the kernel then merges its own splits).
extern "C" int fd_attention_ext(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                const int* block_table, int max_blocks, int num_blocks, int block_size,
                                const int* tok_row, const int* row_slot, const int* row_q_start,
                                const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                                int max_q_len, int n_q, int n_kv, int d, float scale, int window, int dv, int chunk,
                                int n_splits, int split_len, float* scratch, int* status, float softcap, int keep_first,
                                const float* sink, int v_rep, int out_f32, int use_mma, int* counters,
                                cudaStream_t stream) {
    return attention_impl(q, k_pool, v_pool, out, dtype, block_table, max_blocks, num_blocks, block_size, tok_row,
                          row_slot, row_q_start, row_q_len, row_ctx_len, n_rows, T, max_q_len, n_q, n_kv, d, scale,
                          window, dv, chunk, n_splits, split_len, scratch, counters, status, 0, stream, nullptr, 0,
                          softcap, keep_first, sink, v_rep, out_f32, use_mma);
}

// o [T, n_q, n_kv, dv] float, mix [n_q, n_q] float; out (dtype 0 float32, 1 bfloat16): pointer to the first output
// column, rows of ld_out elements.
extern "C" int fd_attn_head_mix(const float* o, const float* mix, void* out, int ld_out, int dtype, int T, int n_q,
                                int n_kv, int dv, float scale, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(n_kv > 0 && n_q % n_kv == 0 && T <= 65535, -2, "attn_head_mix: %d heads on %d, %d tokens", n_q, n_kv, T);
    const size_t staged = (size_t)(n_q * dv + n_q / n_kv * n_q) * sizeof(float);
    if (dv % 4 == 0 && staged <= 48 * 1024 && (uintptr_t)o % 16 == 0) {
        const int work = n_q / n_kv * dv;
        const dim3 sgrid(n_kv, T), sblock(work >= 256 ? 256 : (work + 31) / 32 * 32);
        if (dtype == 0)
            return launch("attn_head_mix", attn_head_mix_staged_kernel<float>, sgrid, sblock, staged, stream, dim3(1, 1, 1), o,
                          mix, (float*)out, ld_out, n_q, n_kv, dv, scale);
        return launch("attn_head_mix", attn_head_mix_staged_kernel<bf16>, sgrid, sblock, staged, stream, dim3(1, 1, 1), o, mix,
                      (bf16*)out, ld_out, n_q, n_kv, dv, scale);
    }
    const dim3 grid(n_q, T);
    const int threads = dv >= 128 ? 128 : (dv + 31) / 32 * 32;
    if (dtype == 0)
        return launch("attn_head_mix", attn_head_mix_kernel<float>, grid, dim3(threads), 0, stream, dim3(1, 1, 1), o, mix,
                      (float*)out, ld_out, n_q, n_kv, dv, scale);
    return launch("attn_head_mix", attn_head_mix_kernel<bf16>, grid, dim3(threads), 0, stream, dim3(1, 1, 1), o, mix,
                  (bf16*)out, ld_out, n_q, n_kv, dv, scale);
}
