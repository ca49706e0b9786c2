// Routed feed-forward (mixture of experts), all decisions on the device:
//
//  * moe_route: per token, router logits in float (one output per warp pass, k in
//    lane order), scores = softmax over all router outputs or a sigmoid of each,
//    the `top` largest of score + correction (ties: the lower index) - by option
//    only among the best groups of neighbouring outputs, a group ranking by the
//    sum of its two largest score + correction - and as weights the chosen
//    scores over their sum, or the chosen scores times a constant;
//  * moe_align: the (token, choice) pairs that go to an expert with weights,
//    grouped by expert, each group padded to whole row tiles, with the expert of
//    every tile and the number of tiles;
//  * moe_gemm: one CTA per (row tile, column tile): rows gathered through the
//    grouping, the tile's expert's matrix; epilogue relu^2 into the grouped
//    activations, or plain rows for the combine.  float32: CUDA cores, k ascending
//    in one fmaf chain per output (no bit depends on what else is in the step);
//    bfloat16: tensor cores (mma.m16n8k16, float accumulators, cp.async ring of
//    three 64-deep k-blocks, swizzled tiles), row tiles of 32 for steps of few
//    tokens and of 128 for prompts;
//  * moe_combine: per token, sum over its choices of weight * (expert row, or the
//    token's own input for an identity expert), plus the shared expert's row.
//
// Router outputs e >= n_experts are identity experts: they have no weights and
// pass their input on.
#include <math.h>

#include "mma_utils.cuh"

namespace fd {

constexpr int ROUTE_THREADS = 1024;     // a warp per router output when the kernel makes the logits itself (one warp selects)
constexpr int MOE_MT = 32;          // rows of a tile
constexpr int MOE_NT = 64;          // columns of a tile
constexpr int MOE_KT = 32;          // k step
constexpr int MOE_THREADS = 256;

// A CTA takes one token.  `logits` null: the CTA computes the token's router logits itself (x row in shared memory as
// float, a warp per output, 16-byte loads, lanes over k); else they are read from logits [T, n_out] (float, made by a
// matrix product) and only the selection runs.
template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ logits,
                 const float* __restrict__ correction, const float* __restrict__ bias, int* __restrict__ ids,
                 float* __restrict__ wts, int H, int n_out, int top, int sigmoid_scores, int n_groups, int keep_groups,
                 int renorm, float weight_scale) {
    // [n_out] logits, then scores; [n_out] choice scores; [n_groups] the groups' ranks; [H] the row
    extern __shared__ __align__(16) float z_s[];
    float* c_s = z_s + n_out;
    float* g_s = c_s + n_out;
    float* x_s = g_s + ((n_groups + 3) & ~3);
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (logits != nullptr) {
        for (int o = threadIdx.x; o < n_out; o += blockDim.x)
            z_s[o] = logits[(size_t)t * n_out + o] + (bias != nullptr ? bias[o] : 0.f);
    } else {
        const T* xr = x + (size_t)t * H;
        for (int k = threadIdx.x; k < H; k += blockDim.x) x_s[k] = to_float(xr[k]);
        __syncthreads();
        constexpr int VEC = 16 / sizeof(T);
        const bool vec = H % VEC == 0 && (uintptr_t)w % 16 == 0;
        for (int o = warp; o < n_out; o += blockDim.x >> 5) {
            const T* wr = w + (size_t)o * H;
            float acc = 0.f;
            if (vec) {
#pragma unroll 8
                for (int c = lane; c < H / VEC; c += 32) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(wr + c * VEC);
                    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) acc = fmaf(to_float(e[j]), x_s[c * VEC + j], acc);
                }
            } else {
                for (int k = lane; k < H; k += 32) acc = fmaf(to_float(wr[k]), x_s[k], acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) z_s[o] = acc + (bias != nullptr ? bias[o] : 0.f);
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (sigmoid_scores) {
        for (int o = lane; o < n_out; o += 32) {
            const float s = 1.f / (1.f + expf(-z_s[o]));
            z_s[o] = s;
            c_s[o] = s + (correction != nullptr ? correction[o] : 0.f);
        }
    } else {
        float m = -INFINITY;
        for (int o = lane; o < n_out; o += 32) m = fmaxf(m, z_s[o]);
        m = warp_max(m);
        float sum = 0.f;
        for (int o = lane; o < n_out; o += 32) {
            const float e = expf(z_s[o] - m);
            z_s[o] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        for (int o = lane; o < n_out; o += 32) {
            const float s = z_s[o] / sum;
            z_s[o] = s;
            c_s[o] = s + (correction != nullptr ? correction[o] : 0.f);
        }
    }
    __syncwarp();
    if (n_groups > 1 && keep_groups < n_groups) {
        // a group's rank: the sum of its two largest choice scores (of its one, if it has one member); outputs of groups
        // outside the best `keep_groups` (ties: the lower group) cannot be chosen
        const int per = n_out / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;
            for (int o = g * per; o < (g + 1) * per; ++o) {
                const float v = c_s[o];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            g_s[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        for (int g = lane; g < n_groups; g += 32) {
            const float mine = g_s[g];
            int ahead = 0;
            for (int o = 0; o < n_groups; ++o) ahead += (g_s[o] > mine) || (g_s[o] == mine && o < g);
            if (ahead >= keep_groups)
                for (int o = g * per; o < (g + 1) * per; ++o) c_s[o] = -INFINITY;
        }
        __syncwarp();
    }
    float chosen_sum = 0.f;
    for (int c = 0; c < top; ++c) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int o = lane; o < n_out; o += 32) {
            const float v = c_s[o];
            if (v > best) { best = v; bi = o; }          // ascending o: the lower index wins a tie
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                     // every score NaN: keep the indices in range
        if (lane == 0) {
            ids[(size_t)t * top + c] = bi;
            c_s[bi] = -INFINITY;
        }
        chosen_sum += z_s[bi];
        __syncwarp();
    }
    const float inv = renorm ? 1.f / (chosen_sum + 1e-20f) : weight_scale;
    for (int c = lane; c < top; c += 32) wts[(size_t)t * top + c] = z_s[ids[(size_t)t * top + c]] * inv;
}

// One CTA.  ids [P] router outputs of the P = tokens * top pairs.  Leaves pair_pos [P] (row of the pair in the grouped
// order, -1 for an identity expert), sorted_pair [cap] (pair of a grouped row, -1 for padding), tile_expert [cap / MT]
// and n_tiles.
__global__ void moe_align_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ pair_pos,
                                 int* __restrict__ sorted_pair, int* __restrict__ tile_expert, int* __restrict__ n_tiles,
                                 int cap, int MT) {
    extern __shared__ int a_s[];           // [E] counts, [E] offsets, [E] fill
    int* cnt = a_s;
    int* off = a_s + E;
    int* fill = a_s + 2 * E;
    __shared__ int total_s;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = run;
            const int tiles = (cnt[e] + MT - 1) / MT;
            for (int i = 0; i < tiles; ++i) tile_expert[run / MT + i] = e;
            run += tiles * MT;
        }
        total_s = run;
        *n_tiles = run / MT;
    }
    __syncthreads();
    const int total = min(total_s, cap);
    for (int i = threadIdx.x; i < total; i += blockDim.x) sorted_pair[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        int pos = -1;
        if (e >= 0 && e < E) {
            pos = off[e] + atomicAdd(&fill[e], 1);
            if (pos < cap) sorted_pair[pos] = p; else pos = -1;
        }
        pair_pos[p] = pos;
    }
}

// MODE 0: a[row] = x[sorted_pair[row] / top], out = relu(acc)^2 as T into act [cap, N]
// MODE 1: a[row] = act[row],                  out = acc as T into y [cap, N]
// MODE 2: a[row] = x[sorted_pair[row] / top], out = acc as T into [cap, N] (an activation kernel follows)
// MODE 3: a[row] = x[sorted_pair[row] / top], w rows in tiles of 8 gate + 8 up rows, out [cap, N / 2] =
//         gated_value(act; 2 = clamped swish with `limit`) of each gate / up pair
template <typename T, int MODE>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w, void* __restrict__ out,
                const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert,
                const int* __restrict__ n_tiles, int top, int N, int K, float limit, int act) {
    const int tile = blockIdx.y;
    if (tile >= *n_tiles) return;
    __shared__ float a_s[MOE_MT][MOE_KT + 1];
    __shared__ float b_s[MOE_NT][MOE_KT + 1];
    __shared__ int row_s[MOE_MT];
    const int e = tile_expert[tile];
    const int n0 = blockIdx.x * MOE_NT;
    const int tid = threadIdx.x;
    if (tid < MOE_MT) {
        const int pr = sorted_pair[tile * MOE_MT + tid];
        row_s[tid] = pr < 0 ? -1 : (MODE != 1 ? pr / top : tile * MOE_MT + tid);
    }
    __syncthreads();
    const T* we = w + (size_t)e * N * K;
    const int ty = tid / 16, tx = tid % 16;        // rows 2 ty, 2 ty + 1; columns tx + 16 j
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += MOE_KT) {
        for (int i = tid; i < MOE_MT * MOE_KT; i += MOE_THREADS) {
            const int r = i / MOE_KT, kk = i - r * MOE_KT;
            const int src = row_s[r];
            a_s[r][kk] = (src >= 0 && k0 + kk < K) ? to_float(a[(size_t)src * K + k0 + kk]) : 0.f;
        }
        for (int i = tid; i < MOE_NT * MOE_KT; i += MOE_THREADS) {
            const int c = i / MOE_KT, kk = i - c * MOE_KT;
            b_s[c][kk] = (n0 + c < N && k0 + kk < K) ? to_float(we[(size_t)(n0 + c) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < MOE_KT; ++kk) {
            const float a0 = a_s[2 * ty][kk], a1 = a_s[2 * ty + 1][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = b_s[tx + 16 * j][kk];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
        __syncthreads();
    }
    if (MODE == 3) {
        // a tile of 16 columns is 8 gate + 8 up values: the thread 8 columns on holds this thread's partner
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, acc[i][j], 8);
                const int r = 2 * ty + i, c = n0 + 16 * j + tx;
                if (tx < 8 && row_s[r] >= 0 && c + 8 < N)
                    static_cast<T*>(out)[(size_t)(tile * MOE_MT + r) * (N >> 1) + ((n0 + 16 * j) >> 1) + tx] =
                        from_float<T>(gated_value(act, acc[i][j], other, limit));
            }
        return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = 2 * ty + i;
        if (row_s[r] < 0) continue;
        const size_t orow = (size_t)(tile * MOE_MT + r) * N;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx + 16 * j;
            if (c >= N) continue;
            if (MODE == 0) {
                const float v = fmaxf(acc[i][j], 0.f);
                static_cast<T*>(out)[orow + c] = from_float<T>(v * v);
            } else {
                static_cast<T*>(out)[orow + c] = from_float<T>(acc[i][j]);
            }
        }
    }
}


// The same product on the tensor cores for bfloat16 (K a multiple of 8).  A CTA of WM x WN warps takes BM grouped rows
// and BN columns; a warp a (BM / WM) x (BN / WN) part of it.
template <int BM, int BN, int WM, int WN, int MODE>
__global__ void __launch_bounds__(WM * WN * 32)
moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, void* __restrict__ out,
                    const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert,
                    const int* __restrict__ n_tiles, int top, int N, int K, float limit, int act) {
    constexpr int THREADS = WM * WN * 32, BK = 64, STAGES = 3;
    constexpr int TM = BM / WM, TN = BN / WN, MI = TM / 16, NI = TN / 8;
    static_assert(TM % 16 == 0 && TN % 16 == 0, "a warp takes whole 16 x 16 parts");
    const int tile = blockIdx.y;
    if (tile >= *n_tiles) return;
    extern __shared__ __align__(128) unsigned char mm_smem[];
    unsigned char* a_s = mm_smem;                                   // [STAGES][BM][64] bf16, swizzled
    unsigned char* b_s = a_s + STAGES * BM * BK * 2;                // [STAGES][BN][64]
    int* row_s = reinterpret_cast<int*>(b_s + STAGES * BN * BK * 2);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WN, wn = warp % WN;
    const int n0 = blockIdx.x * BN;
    for (int i = tid; i < BM; i += THREADS) {
        const int pr = sorted_pair[tile * BM + i];
        row_s[i] = pr < 0 ? -1 : (MODE != 1 ? pr / top : tile * BM + i);
    }
    __syncthreads();
    const __nv_bfloat16* we = w + (size_t)tile_expert[tile] * N * K;
    const int nkb = (K + BK - 1) / BK;
    auto issue = [&](int kb, int stage) {
        unsigned char* as = a_s + stage * BM * BK * 2;
        unsigned char* bs = b_s + stage * BN * BK * 2;
        for (int c = tid; c < BM * 8; c += THREADS) {
            const int r = c >> 3, cc = c & 7;
            const int k = kb * BK + cc * 8;
            const int src = row_s[r];
            const bool ok = src >= 0 && k < K;
            cp_async16(smem_u32(as + swz<BK>(r, cc)), ok ? a + (size_t)src * K + k : a, ok ? 16 : 0);
        }
        for (int c = tid; c < BN * 8; c += THREADS) {
            const int r = c >> 3, cc = c & 7;
            const int k = kb * BK + cc * 8;
            const bool ok = n0 + r < N && k < K;
            cp_async16(smem_u32(bs + swz<BK>(r, cc)), ok ? we + (size_t)(n0 + r) * K + k : we, ok ? 16 : 0);
        }
    };
    float acc[MI][NI][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nkb) issue(s, s);
        cp_async_commit();
    }
    const int mi8 = lane >> 3;
    for (int kb = 0; kb < nkb; ++kb) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();              // block kb has landed for everyone, and everyone is done with block kb - 1
        if (kb + STAGES - 1 < nkb) issue(kb + STAGES - 1, (kb + STAGES - 1) % STAGES);
        cp_async_commit();
        const unsigned char* as = a_s + (kb % STAGES) * BM * BK * 2;
        const unsigned char* bs = b_s + (kb % STAGES) * BN * BK * 2;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            uint32_t af[MI][4];
#pragma unroll
            for (int i = 0; i < MI; ++i) {
                const int r = wm * TM + i * 16 + (mi8 & 1) * 8 + (lane & 7);
                ldmatrix_x4(smem_u32(as + swz<BK>(r, ks * 2 + (mi8 >> 1))), af[i][0], af[i][1], af[i][2], af[i][3]);
            }
#pragma unroll
            for (int jp = 0; jp < NI / 2; ++jp) {
                const int r = wn * TN + jp * 16 + (mi8 >> 1) * 8 + (lane & 7);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(smem_u32(bs + swz<BK>(r, ks * 2 + (mi8 & 1))), b0, b1, b2, b3);
#pragma unroll
                for (int i = 0; i < MI; ++i) {
                    mma_bf16(acc[i][2 * jp], af[i][0], af[i][1], af[i][2], af[i][3], b0, b1);
                    mma_bf16(acc[i][2 * jp + 1], af[i][0], af[i][1], af[i][2], af[i][3], b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int r = wm * TM + i * 16 + (lane >> 2) + hh * 8;
            if (row_s[r] < 0) continue;
            if (MODE == 3) {
                // columns j * 8 .. of even j are gate values, those of j + 1 the up values of the same outputs
                __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out) + (size_t)(tile * BM + r) * (N >> 1);
#pragma unroll
                for (int j = 0; j < NI; j += 2) {
                    const int cg = n0 + wn * TN + j * 8;
                    if (cg + 16 > N) continue;
                    *reinterpret_cast<__nv_bfloat162*>(o + (cg >> 1) + (lane & 3) * 2) =
                        __floats2bfloat162_rn(gated_value(act, acc[i][j][hh * 2], acc[i][j + 1][hh * 2], limit),
                                              gated_value(act, acc[i][j][hh * 2 + 1], acc[i][j + 1][hh * 2 + 1], limit));
                }
                continue;
            }
            const size_t orow = (size_t)(tile * BM + r) * N;
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                const int c = n0 + wn * TN + j * 8 + (lane & 3) * 2;
                float v0 = acc[i][j][hh * 2], v1 = acc[i][j][hh * 2 + 1];
                if (MODE == 0) {
                    v0 = fmaxf(v0, 0.f); v0 *= v0;
                    v1 = fmaxf(v1, 0.f); v1 *= v1;
                }
                {
                    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out) + orow + c;
                    if (c + 1 < N && (N & 1) == 0) *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(v0, v1);
                    else { if (c < N) o[0] = __float2bfloat16_rn(v0); if (c + 1 < N) o[1] = __float2bfloat16_rn(v1); }
                }
            }
        }
}

template <int BM, int BN, int WM, int WN, int MODE>
static int launch_moe_mma(const void* a, const void* w, void* out, const int* sorted_pair, const int* tile_expert,
                          const int* n_tiles, int cap, int top, int N, int K, float limit, int act, cudaStream_t stream) {
    auto k = moe_gemm_mma_kernel<BM, BN, WM, WN, MODE>;
    const size_t smem = (size_t)3 * (BM + BN) * 64 * 2 + BM * sizeof(int);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-3, "moe_gemm: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((N + BN - 1) / BN, cap / BM);
    FD_REQUIRE(grid.y <= 65535, -2, "moe_gemm: %d row tiles are too many", (int)grid.y);
    return launch("moe_gemm", k, grid, dim3(WM * WN * 32), smem, stream, dim3(1, 1, 1), (const __nv_bfloat16*)a,
                  (const __nv_bfloat16*)w, out, sorted_pair, tile_expert, n_tiles, top, N, K, limit, act);
}

// xs[row] = x[sorted_pair[row] / top] for the grouped rows that exist, zeros for the padding rows among them: the
// grouped rows as one contiguous matrix, for products that read their operands through tensor maps.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ xs,
                                  const int* __restrict__ sorted_pair, const int* __restrict__ n_tiles, int mt, int top,
                                  int K8) {
    const int row = blockIdx.x;
    if (row >= *n_tiles * mt) return;
    const int pr = sorted_pair[row];
    const uint4* src = pr < 0 ? nullptr : reinterpret_cast<const uint4*>(x) + (size_t)(pr / top) * K8;
    uint4* dst = reinterpret_cast<uint4*>(xs) + (size_t)row * K8;
    for (int c = threadIdx.x; c < K8; c += blockDim.x) dst[c] = src != nullptr ? src[c] : make_uint4(0, 0, 0, 0);
}

__device__ __forceinline__ void load4(const float* p, float v[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float v[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

constexpr int COMBINE_MAX_TOP = 64;       // choices per token whose rows, weights and places the combine keeps in shared memory

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ shared,
                                   const int* __restrict__ ids, const float* __restrict__ wts,
                                   const int* __restrict__ pair_pos, T* __restrict__ out, int H, int top, int E) {
    __shared__ int pos_s[COMBINE_MAX_TOP];        // row of y, -1: the token's own input (identity), -2: nothing
    __shared__ float w_s[COMBINE_MAX_TOP];
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < top; c += blockDim.x) {
        const size_t p = t * top + c;
        w_s[c] = wts[p];
        const int pp = pair_pos[p];
        pos_s[c] = ids[p] >= E ? -1 : (pp >= 0 ? pp : -2);
    }
    __syncthreads();
    // four columns per thread where the rows allow 16-byte loads of y
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float xv[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 4; ++j) xv[j] = to_float(x[t * H + i + j]);
            for (int c = 0; c < top; ++c) {
                const int pos = pos_s[c];
                const float wgt = w_s[c];
                if (pos == -1) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[j] = fmaf(wgt, xv[j], acc[j]);
                } else if (pos >= 0) {
                    float v[4];
                    load4(y + (size_t)pos * H + i, v);
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[j] = fmaf(wgt, v[j], acc[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (shared != nullptr) acc[j] += to_float(shared[t * H + i + j]);
                out[t * H + i + j] = from_float<T>(acc[j]);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < top; ++c) {
            const int pos = pos_s[c];
            if (pos == -1) acc = fmaf(w_s[c], to_float(x[t * H + i]), acc);
            else if (pos >= 0) acc = fmaf(w_s[c], to_float(y[(size_t)pos * H + i]), acc);
        }
        if (shared != nullptr) acc += to_float(shared[t * H + i]);
        out[t * H + i] = from_float<T>(acc);
    }
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// Rows of a tile of the grouped products: 32 on the CUDA cores (float32) and for steps of few tokens, 128 for
// bfloat16 steps with many rows per expert.
extern "C" int fd_moe_tile_rows(int dtype, int rows_per_expert) { return dtype == 1 && rows_per_expert >= 96 ? 128 : MOE_MT; }

// x [T, H] and w [n_out, H] of type dtype (0 float32, 1 bfloat16), or logits [T, n_out] float made from them by a
// matrix product (then x and w are not read); correction [n_out] float or null; ids [T, top] int32 and wts [T, top]
// float come back.
// bias [n_out] float or null: added to the logits before the softmax (correction only shifts the choice).
extern "C" int fd_moe_route(const void* x, const void* w, int dtype, const float* logits, const float* correction,
                            const float* bias, int* ids, float* wts, int T, int H, int n_out, int top,
                            int sigmoid_scores, int n_groups, int keep_groups, int renorm, float weight_scale,
                            cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(n_groups >= 1 && n_out % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups &&
               (long long)keep_groups * (n_out / n_groups) >= top, -2,
               "moe_route: %d of %d groups of %d router outputs for %d choices", keep_groups, n_groups, n_out, top);
    FD_REQUIRE(n_out >= 1 && top >= 1 && top <= n_out && n_out <= 4096, -2,
               "moe_route: %d choices of %d router outputs (at most 4096)", top, n_out);
    const size_t smem = (2 * (size_t)n_out + ((n_groups + 3) & ~3) + (logits ? 0 : H)) * sizeof(float);
    FD_REQUIRE(smem <= 48 * 1024, -2, "moe_route: a row of %d and %d outputs need %zu bytes of shared memory (max 48 KB); "
               "give the logits", H, n_out, smem);
    const int threads = logits != nullptr ? 32 : (n_out >= 32 ? ROUTE_THREADS : ((n_out + 7) / 8 * 8) * 32);
    if (dtype == 0)
        return launch("moe_route", moe_route_kernel<float>, dim3(T), dim3(threads), smem, stream, dim3(1, 1, 1),
                      (const float*)x, (const float*)w, logits, correction, bias, ids, wts, H, n_out, top, sigmoid_scores,
                      n_groups, keep_groups, renorm, weight_scale);
    return launch("moe_route", moe_route_kernel<bf16>, dim3(T), dim3(threads), smem, stream, dim3(1, 1, 1),
                  (const bf16*)x, (const bf16*)w, logits, correction, bias, ids, wts, H, n_out, top, sigmoid_scores, n_groups,
                  keep_groups, renorm, weight_scale);
}

// cap: rows of the grouped buffers, at least P rounded up to whole tiles plus one tile per expert.
// mt: rows of a tile (32 or 128).
extern "C" int fd_moe_align(const int* ids, int P, int E, int* pair_pos, int* sorted_pair, int* tile_expert,
                            int* n_tiles, int cap, int mt, cudaStream_t stream) {
    FD_REQUIRE(E >= 1 && E <= 4096, -2, "moe_align: %d experts (1..4096)", E);
    FD_REQUIRE(mt == 32 || mt == 128, -2, "moe_align: tiles of %d rows (32 or 128)", mt);
    const long long worst = (long long)P + (long long)(E < P ? E : P) * (mt - 1);     // every group's last tile nearly empty
    FD_REQUIRE(cap % mt == 0 && (long long)cap >= (worst + mt - 1) / mt * mt, -2,
               "moe_align: %d grouped rows cannot hold %d pairs of %d experts", cap, P, E);
    return launch("moe_align", moe_align_kernel, dim3(1), dim3(1024), 3 * (size_t)E * sizeof(int), stream, dim3(1, 1, 1),
                  ids, P, E, pair_pos, sorted_pair, tile_expert, n_tiles, cap, mt);
}

// mode 0: a = x [T, K], out = act [cap, N] (dtype) = relu(x W_e^T)^2;  mode 1: a = act [cap, K], out = y [cap, N] (dtype);
// mode 2: a = x [T, K], out [cap, N] (dtype) = x W_e^T.
// w [E, N, K].
// mt: the tile rows the grouping was made with.
// mode 3: a = x [T, K], w rows in tiles of 8 gate + 8 up, out [cap, N / 2] = gated_value(act) of each gate / up pair:
// act 0 SiLU(gate) up, 1 tanh-GELU(gate) up, 2 clamped swish of gate times (up + 1) with `limit`.
extern "C" int fd_moe_gemm(const void* a, const void* w, void* out, int dtype, int mode, const int* sorted_pair,
                           const int* tile_expert, const int* n_tiles, int cap, int mt, int top, int N, int K,
                           float limit, int act, cudaStream_t stream) {
    if (cap == 0) return 0;
    FD_REQUIRE(act >= 0 && act <= 2, -2, "moe_gemm: unknown gated activation %d", act);
    FD_REQUIRE(cap % mt == 0 && N > 0 && K > 0 && mode >= 0 && mode <= 3 && (mode != 3 || N % 16 == 0), -2,
               "moe_gemm: bad sizes or mode (the gated form needs N, twice the outputs, to be a multiple of 16)");
    if (dtype == 1 && K % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0) {
        if (mt == 128) {
            if (mode == 0) return launch_moe_mma<128, 128, 2, 4, 0>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
            if (mode == 2) return launch_moe_mma<128, 128, 2, 4, 2>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
            if (mode == 3) return launch_moe_mma<128, 128, 2, 4, 3>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
            return launch_moe_mma<128, 128, 2, 4, 1>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
        }
        if (mt == 32) {
            if (mode == 0) return launch_moe_mma<32, 64, 1, 4, 0>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
            if (mode == 2) return launch_moe_mma<32, 64, 1, 4, 2>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
            if (mode == 3) return launch_moe_mma<32, 64, 1, 4, 3>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
            return launch_moe_mma<32, 64, 1, 4, 1>(a, w, out, sorted_pair, tile_expert, n_tiles, cap, top, N, K, limit, act, stream);
        }
    }
    FD_REQUIRE(mt == MOE_MT, -2, "moe_gemm: the CUDA-core product takes tiles of %d rows, not %d", MOE_MT, mt);
    dim3 grid((N + MOE_NT - 1) / MOE_NT, cap / MOE_MT);
    FD_REQUIRE(grid.y <= 65535, -2, "moe_gemm: %d row tiles are too many", (int)grid.y);
#define FD_MG(T_, M_)                                                                                                \
    return launch("moe_gemm", moe_gemm_kernel<T_, M_>, grid, dim3(MOE_THREADS), 0, stream, dim3(1, 1, 1), (const T_*)a, \
                  (const T_*)w, out, sorted_pair, tile_expert, n_tiles, top, N, K, limit, act)
    if (dtype == 0) { if (mode == 0) FD_MG(float, 0); if (mode == 2) FD_MG(float, 2); if (mode == 3) FD_MG(float, 3); FD_MG(float, 1); }
    if (mode == 0) FD_MG(bf16, 0);
    if (mode == 2) FD_MG(bf16, 2);
    if (mode == 3) FD_MG(bf16, 3);
    FD_MG(bf16, 1);
#undef FD_MG
}

// xs [cap, K] <- the rows of x [T, K] (bfloat16, K a multiple of 8) in grouped order.
extern "C" int fd_moe_gather(const void* x, void* xs, const int* sorted_pair, const int* n_tiles, int cap, int mt,
                             int top, int K, cudaStream_t stream) {
    if (cap == 0) return 0;
    FD_REQUIRE(K % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)xs % 16 == 0, -2, "moe_gather: rows of %d need 16-byte chunks", K);
    return launch("moe_gather", moe_gather_kernel, dim3(cap), dim3(K / 8 >= 256 ? 256 : 128), 0, stream, dim3(1, 1, 1),
                  (const bf16*)x, (bf16*)xs, sorted_pair, n_tiles, mt, top, K / 8);
}

extern "C" int fd_moe_combine(const void* y, const void* x, const void* shared, const int* ids, const float* wts,
                              const int* pair_pos, void* out, int dtype, int T, int H, int top, int E,
                              cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(top <= COMBINE_MAX_TOP, -2, "moe_combine: %d choices per token (at most %d)", top, COMBINE_MAX_TOP);
    FD_REQUIRE((uintptr_t)y % 16 == 0, -2, "moe_combine: the experts' rows must be 16-byte aligned");
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == 0)
        return launch("moe_combine", moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                      (const float*)y, (const float*)x, (const float*)shared, ids, wts, pair_pos, (float*)out, H, top, E);
    return launch("moe_combine", moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                  (const bf16*)y, (const bf16*)x, (const bf16*)shared, ids, wts, pair_pos, (bf16*)out, H, top, E);
}
