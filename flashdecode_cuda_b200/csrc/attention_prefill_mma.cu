// Prompt attention (many new tokens per sequence) over the paged bfloat16
// cache on the tensor cores: causal, grouped-query, variable lengths, optional
// sliding window, and the new tokens may continue a cached prefix.
//
// A CTA takes 64 consecutive query tokens of one sequence and one query head;
// each of its 4 warps owns 16 query rows.  Keys and values of the head's KV
// head stream through shared memory in tiles of 64 tokens, gathered from the
// block table with cp.async (double buffered, XOR-swizzled for ldmatrix):
//     S[16, 64] = Q[16, D] K^T      O[16, D] += P[16, 64] V[64, D]
// with the online softmax (float, base 2) between the two products, as in the
// decode kernel.  Tiles start at multiples of 64 in absolute position, so a
// query's sums do not depend on what else is in the batch.
//
// The EXT form of the kernel has the options of the CUDA-core kernel as well: scores capped by a tanh, a window that
// also keeps the first positions (the key tiles between those and the window's start are not visited), a keyless term
// per head in the softmax denominator, and weights that are applied to every value head (a CTA takes VR of them at a
// time, its scores and softmax worked out once; out [T, n_q, v_rep, D]), written as float on request.  Its weights reach the second product as a sum of two
// bfloat16 numbers (the rounded weight and what the rounding took away), so they carry 16 bits of mantissa and not 8.
#include <math.h>

#include "attention.cuh"
#include "mma_utils.cuh"

namespace fd {

constexpr int PM_WARPS = 4;
constexpr int PM_THREADS = PM_WARPS * 32;
constexpr int PM_BM = 64;     // query rows per CTA
constexpr int PM_BN = 64;     // keys per tile

template <int D, bool EXT, int VR>
__global__ void __launch_bounds__(PM_THREADS)
attn_prefill_mma_kernel(const AttnParams p) {
    constexpr int CPR = D / 8;                      // 16-byte chunks per row
    constexpr int TILE_BYTES = PM_BN * D * 2;
    // the last query tiles of a sequence see the most keys: schedule them first, so that the
    // short tiles fill the tail of the launch instead of the long ones
    const int tile = gridDim.x - 1 - blockIdx.x, b = blockIdx.z;
    // grid.y = query head * groups of VR value heads + group: the CTA's weights meet VR value heads, scores worked out once
    const int v_groups = EXT ? p.v_rep / VR : 1;
    const int h = EXT ? blockIdx.y / v_groups : blockIdx.y;                  // query head
    const int vhi = EXT ? (blockIdx.y - h * v_groups) * VR : 0;              // first of its value heads
    const int slot = p.row_slot[b];
    if (slot < 0) return;
    const int q_len = p.row_q_len[b];
    if (tile * PM_BM >= q_len) return;
    const int ctx = p.row_ctx_len[b];
    const int tok0 = p.row_q_start[b] + tile * PM_BM;
    const int nq = min(PM_BM, q_len - tile * PM_BM);
    const int kvh = h / p.G;
    const int vh = (EXT && p.v_rep > 1) ? vhi : kvh;                         // the (first) head whose values the weights meet
    const int keep = (EXT && p.window > 0) ? p.keep_first : 0;               // first positions that stay visible
    const float softcap = p.softcap;
    const int p_first = ctx + tile * PM_BM;          // position of this CTA's first query
    const int hi = p_first + nq;                      // keys 0 .. last query position
    const int chunk = p.chunk;        // > 0: a query sees the keys of its own chunk of this many positions only
    const int lo = max(p.window > 0 ? max(0, p_first - p.window + 1) : 0, chunk > 0 ? (p_first / chunk) * chunk : 0);

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                        // [64][D]
    unsigned char* k_s = q_s + PM_BM * D * 2;         // [2][64][D]
    unsigned char* v_s = k_s + 2 * TILE_BYTES;        // [2][VR][64][D]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* qg = static_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(p.k_pool);
    const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(p.v_pool);
    const int bs = p.block_size;
    const int bs_shift = (bs & (bs - 1)) == 0 ? __ffs(bs) - 1 : -1;     // block sizes that are powers of two: shift and mask

    // queries of the tile (rows beyond nq as zeros)
#pragma unroll
    for (int i = 0; i < PM_BM * CPR / PM_THREADS; ++i) {
        const int c = i * PM_THREADS + tid;
        const int r = c / CPR, cc = c - r * CPR;
        const bool ok = r < nq;
        const __nv_bfloat16* src = ok ? qg + ((size_t)(tok0 + r) * p.n_q + h) * D + cc * 8 : qg;
        cp_async16(smem_u32(q_s + swz<D>(r, cc)), src, ok ? 16 : 0);
    }
    auto issue = [&](int t0, int stage) {
        unsigned char* ks = k_s + stage * TILE_BYTES;
        unsigned char* vs = v_s + stage * VR * TILE_BYTES;
#pragma unroll
        for (int i = 0; i < PM_BN * CPR / PM_THREADS; ++i) {
            const int c = i * PM_THREADS + tid;
            const int r = c / CPR, cc = c - r * CPR;
            const int t = t0 + r;
            const __nv_bfloat16* ksrc = kp;
            const __nv_bfloat16* vsrc = vp;
            size_t v_head_step = 0;                   // elements from one value head's row to the next one's
            int bytes = 0;
            if ((t >= lo || (EXT && t < keep)) && t < hi) {
                const int col = bs_shift >= 0 ? t >> bs_shift : t / bs;
                const int in_blk = bs_shift >= 0 ? t & (bs - 1) : t - col * bs;
                const int blk = p.block_table[(size_t)slot * p.max_blocks + col];
                if (blk < 0 || blk >= p.num_blocks) {
                    set_status(p.status, STATUS_BAD_BLOCK);
                } else {
                    const size_t off = (((size_t)blk * p.n_kv + kvh) * bs + in_blk) * D + cc * 8;
                    ksrc = kp + off;
                    vsrc = EXT ? vp + (((size_t)blk * p.n_kv + vh) * bs + in_blk) * D + cc * 8 : vp + off;
                    v_head_step = (size_t)bs * D;
                    bytes = 16;
                }
            }
            cp_async16(smem_u32(ks + swz<D>(r, cc)), ksrc, bytes);
#pragma unroll
            for (int j = 0; j < VR; ++j)
                cp_async16(smem_u32(vs + j * TILE_BYTES + swz<D>(r, cc)), vsrc + j * v_head_step, bytes);
        }
        cp_async_commit();
    };

    const int t_begin = (lo / PM_BN) * PM_BN;
    // tiles of kept first keys that lie wholly before the window's first tile come first; a kept key in a window tile
    // is loaded and seen there
    const int n_kf = EXT ? min((min(keep, lo) + PM_BN - 1) / PM_BN, t_begin / PM_BN) : 0;
    const int n_tiles = n_kf + (hi - t_begin + PM_BN - 1) / PM_BN;
    auto tile_t0 = [&](int it) { return it < n_kf ? it * PM_BN : t_begin + (it - n_kf) * PM_BN; };
    issue(tile_t0(0), 0);                             // this group also carries the queries

    // head sizes above 128: the query fragments are read from shared memory for every key tile instead of being kept
    // (with the output tile they would not fit the registers)
    constexpr bool Q_REGS = D * VR <= 128;
    uint32_t qf[Q_REGS ? D / 16 : 1][4];
    float o[VR][D / 8][4];
#pragma unroll
    for (int j = 0; j < VR; ++j)
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[j][i][0] = o[j][i][1] = o[j][i][2] = o[j][i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    const float scale_log2 = p.scale * 1.4426950408889634f;
    // capped scores: exponent 2 x log2(e) of the score's x = s * scale / cap, and the cap in base-2 units
    const float cap_in = softcap > 0.f ? 2.f * 1.4426950408889634f * p.scale / softcap : 0.f;
    const float cap_out = softcap * 1.4426950408889634f;
    const int row_a = warp * 16 + (lane >> 2);        // this thread's rows: row_a and row_a + 8
    const int pos_a = p_first + row_a, pos_b = pos_a + 8;
    const int w_first = p_first + warp * 16, w_last = w_first + 15;     // positions of the warp's rows
    // first visible key of this thread's rows and of the warp's first and last row under chunked visibility
    const int cs_a = chunk > 0 ? (pos_a / chunk) * chunk : 0, cs_b = chunk > 0 ? (pos_b / chunk) * chunk : 0;
    const int cs_first = chunk > 0 ? (w_first / chunk) * chunk : 0, cs_last = chunk > 0 ? (w_last / chunk) * chunk : 0;

    for (int it = 0; it < n_tiles; ++it) {
        const int t0 = tile_t0(it);
        if (it + 1 < n_tiles) {
            issue(tile_t0(it + 1), (it + 1) & 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (Q_REGS && it == 0) {
            const int mi = lane >> 3, r = warp * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(smem_u32(q_s + swz<D>(r, ks * 2 + (mi >> 1))), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        const unsigned char* ks_ = k_s + (it & 1) * TILE_BYTES;
        const unsigned char* vs_ = v_s + (it & 1) * VR * TILE_BYTES;
        // a tile wholly in the future of all rows of this warp contributes nothing
        const bool skip = t0 > w_last || (p.window > 0 && t0 + PM_BN - 1 < w_first - p.window + 1 && !(EXT && t0 < keep)) ||
                          t0 + PM_BN - 1 < cs_first;
        if (!skip) {
            float s[PM_BN / 8][4];
#pragma unroll
            for (int i = 0; i < PM_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            {
                const int mi = lane >> 3;
                const int qr = warp * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    uint32_t a0, a1, a2, a3;
                    if (Q_REGS) { a0 = qf[kk][0]; a1 = qf[kk][1]; a2 = qf[kk][2]; a3 = qf[kk][3]; }
                    else ldmatrix_x4(smem_u32(q_s + swz<D>(qr, kk * 2 + (mi >> 1))), a0, a1, a2, a3);
#pragma unroll
                    for (int np = 0; np < PM_BN / 16; ++np) {
                        const int r = np * 16 + (mi >> 1) * 8 + (lane & 7);
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(smem_u32(ks_ + swz<D>(r, kk * 2 + (mi & 1))), b0, b1, b2, b3);
                        mma_bf16(s[np * 2], a0, a1, a2, a3, b0, b1);
                        mma_bf16(s[np * 2 + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
            const bool need_mask = t0 + PM_BN - 1 > w_first || t0 < lo || t0 + PM_BN > hi ||
                                   (p.window > 0 && t0 < w_last - p.window + 1) || t0 < cs_last;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < PM_BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[nt][e] * scale_log2;
                    if (EXT && softcap > 0.f) {
                        // cap * tanh(x) as cap * (1 - 2 / (e^(2x) + 1)), in float: its error stays below 1e-7 of the cap
                        const float ex = exp2f(s[nt][e] * cap_in);
                        v = fmaf(-2.f * cap_out, __fdividef(1.f, ex + 1.f), cap_out);
                    }
                    if (need_mask) {
                        const int t = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int pos = (e >> 1) ? pos_b : pos_a;
                        const bool ok = (t >= lo || (EXT && t < keep)) && t < hi && t <= pos &&
                                        (p.window <= 0 || pos - t < p.window || (EXT && t < keep)) &&
                                        t >= ((e >> 1) ? cs_b : cs_a);
                        if (!ok) v = -INFINITY;
                    }
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
                const float m_new = fmaxf(m_run[hh], mx[hh]);
                alpha[hh] = m_new == -INFINITY ? 1.f : exp2f(m_run[hh] - m_new);
                m_run[hh] = m_new;
            }
            float rs[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < PM_BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = m_run[e >> 1] == -INFINITY ? 0.f : exp2f(s[nt][e] - m_run[e >> 1]);
                    s[nt][e] = pv;
                    rs[e >> 1] += pv;
                }
            l_run[0] = l_run[0] * alpha[0] + rs[0];
            l_run[1] = l_run[1] * alpha[1] + rs[1];
#pragma unroll
            for (int j = 0; j < VR; ++j)
#pragma unroll
                for (int i = 0; i < D / 8; ++i) {
                    o[j][i][0] *= alpha[0]; o[j][i][1] *= alpha[0]; o[j][i][2] *= alpha[1]; o[j][i][3] *= alpha[1];
                }
            {
                const int mi = lane >> 3;
#pragma unroll
                for (int k2 = 0; k2 < PM_BN / 16; ++k2) {
                    const uint32_t pa0 = pack_bf16(s[2 * k2][0], s[2 * k2][1]), pa1 = pack_bf16(s[2 * k2][2], s[2 * k2][3]);
                    const uint32_t pa2 = pack_bf16(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
                    const uint32_t pa3 = pack_bf16(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
                    uint32_t pb0 = 0, pb1 = 0, pb2 = 0, pb3 = 0;        // what rounding to bfloat16 took from the weights
                    if (EXT) {
                        pb0 = pack_bf16_rest(s[2 * k2][0], s[2 * k2][1]); pb1 = pack_bf16_rest(s[2 * k2][2], s[2 * k2][3]);
                        pb2 = pack_bf16_rest(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
                        pb3 = pack_bf16_rest(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
                    }
                    const int r = k2 * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int j = 0; j < VR; ++j)
#pragma unroll
                        for (int np = 0; np < D / 16; ++np) {
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4_trans(smem_u32(vs_ + j * TILE_BYTES + swz<D>(r, np * 2 + (mi >> 1))), b0, b1, b2, b3);
                            mma_bf16(o[j][np * 2], pa0, pa1, pa2, pa3, b0, b1);
                            mma_bf16(o[j][np * 2 + 1], pa0, pa1, pa2, pa3, b2, b3);
                            if (EXT) {
                                mma_bf16(o[j][np * 2], pb0, pb1, pb2, pb3, b0, b1);
                                mma_bf16(o[j][np * 2 + 1], pb0, pb1, pb2, pb3, b2, b3);
                            }
                        }
                }
            }
        }
        __syncthreads();          // everyone is done with this stage before it is refilled
    }

#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    __nv_bfloat16* og = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = row_a + hh * 8;
        if (r >= nq) continue;
        float l = l_run[hh], f = 1.f;
        if (EXT && p.sink != nullptr) {             // one more term in the denominator: exp(sink), no key, no value
            const float sk = p.sink[h] * 1.4426950408889634f, m = m_run[hh];
            const float m2 = fmaxf(m, sk);
            f = m == -INFINITY ? 0.f : exp2f(m - m2);
            l = l * f + exp2f(sk - m2);
        }
        const float inv = l > 0.f ? f / l : 0.f;
#pragma unroll
        for (int j = 0; j < VR; ++j) {
            const size_t orow_i = EXT ? ((size_t)(tok0 + r) * p.n_q + h) * p.v_rep + vhi + j : (size_t)(tok0 + r) * p.n_q + h;
            if (EXT && p.out_f32) {
                float* orow = static_cast<float*>(p.out) + orow_i * D + (lane & 3) * 2;
#pragma unroll
                for (int nt = 0; nt < D / 8; ++nt)
                    *reinterpret_cast<float2*>(orow + nt * 8) = make_float2(o[j][nt][hh * 2] * inv, o[j][nt][hh * 2 + 1] * inv);
                continue;
            }
            __nv_bfloat16* orow = og + orow_i * D + (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < D / 8; ++nt)
                *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8) =
                    __floats2bfloat162_rn(o[j][nt][hh * 2] * inv, o[j][nt][hh * 2 + 1] * inv);
        }
    }
}

template <int D, bool EXT, int VR = 1>
static int launch_pm(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream) {
    constexpr size_t smem = (size_t)(PM_BM + 2 * PM_BN + 2 * VR * PM_BN) * D * 2;
    auto k = attn_prefill_mma_kernel<D, EXT, VR>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-3, "attention: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int q_tiles = (max_q_len + PM_BM - 1) / PM_BM;
    const int heads = EXT ? p.n_q * (p.v_rep / VR) : p.n_q;
    if (heads > 65535 || n_rows > 65535) return 1;
    dim3 grid(q_tiles, heads, n_rows);
    k<<<grid, PM_THREADS, smem, stream>>>(p);
    return check_launch(EXT ? "attention_ext_prefill_mma" : "attention_prefill_mma");
}

int launch_attn_prefill_mma(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream) {
    if (p.n_splits != 1) return 1;
    if (p.d == 128) return launch_pm<128, false>(p, n_rows, max_q_len, stream);
    if (p.d == 64) return launch_pm<64, false>(p, n_rows, max_q_len, stream);
    // wider heads (one cached latent as key and value of many query heads): rows of whole 128-byte swizzle groups
    if (p.d == 256) return launch_pm<256, false>(p, n_rows, max_q_len, stream);
    if (p.d == 192) return launch_pm<192, false>(p, n_rows, max_q_len, stream);
    return 1;
}

// The form with the capped scores, kept first keys, keyless term and repeated value heads; returns 1 for sizes it does
// not take.
int launch_attn_prefill_mma_ext(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream) {
    if (p.n_splits != 1 || p.d != p.dv || p.chunk > 0) return 1;
    // repeated value heads: a CTA takes two of them (four of 64 dimensions), as many as its registers hold outputs for
    if (p.d == 128) return p.v_rep % 2 == 0 ? launch_pm<128, true, 2>(p, n_rows, max_q_len, stream)
                                            : launch_pm<128, true, 1>(p, n_rows, max_q_len, stream);
    if (p.d == 64) return p.v_rep % 4 == 0   ? launch_pm<64, true, 4>(p, n_rows, max_q_len, stream)
                          : p.v_rep % 2 == 0 ? launch_pm<64, true, 2>(p, n_rows, max_q_len, stream)
                                             : launch_pm<64, true, 1>(p, n_rows, max_q_len, stream);
    return 1;
}

}  // namespace fd
