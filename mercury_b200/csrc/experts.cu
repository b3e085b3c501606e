// A feed-forward of routed experts: the router, the plan that sorts a step's (token, choice)
// pairs by expert, the two grouped products and the weighted sum.
//
// Router (float32): s = sigmoid(Wr x); the choice is made on s + correction; the experts form
// equal groups of neighbours, a group's score is the sum of its two largest choice scores,
// only experts of the best `group_keep` groups can be chosen, and of those the `top` with
// the largest choice scores are (ties: the lower index). A chosen expert's weight is
// s * route_scale.
//
// Products: the pairs are sorted by expert and cut into tiles of EX_BM rows that belong to
// one expert each, so that a block reads a tile of that expert's matrix once for all its
// rows. The grid is sized for the most tiles a step of that many pairs can have; blocks
// beyond the step's own count leave at once, so the launch sequence depends on the step's
// shape only. Every output is one sum over k in ascending order, whatever else is in the
// tile: a token's result does not depend on the batch. Each pair's result of the second
// product is kept apart (float32) and a token's pairs are added in the order of the
// router's choice.
#include "common.cuh"

namespace mb {

constexpr int EX_BM = 32;   // rows (token, choice pairs) per tile
constexpr int EX_BN = 64;   // output columns per block
constexpr int EX_BK = 32;   // k per round

// the better of two candidates: larger value, lower index on a tie; index -1 is no candidate
__device__ __forceinline__ void take_better(float& v, int& i, float v2, int i2) {
    if (i2 >= 0 && (i < 0 || v2 > v || (v2 == v && i2 < i))) {
        v = v2;
        i = i2;
    }
}

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
        take_better(v, i, v2, i2);
    }
}

// Router logits: z[t][e] = Wr[e] . x[t] in float32. A block of eight warps takes RT tokens and
// eight experts, one expert a warp: a lane reads its share of the expert's row once and
// multiplies it with the RT tokens' rows (staged in shared memory as float32).
template <typename T, int RT>
__global__ void __launch_bounds__(256)
router_logits_kernel(const T* __restrict__ x, const float* __restrict__ router,
                     float* __restrict__ logits, int tokens, int hidden, int experts) {
    grid_dependency_sync();
    extern __shared__ float x_s[];                 // [RT][hidden]
    const int t0 = blockIdx.x * RT;
    for (int idx = threadIdx.x; idx < RT * hidden; idx += blockDim.x) {
        const int tt = idx / hidden, k = idx - tt * hidden;
        x_s[idx] = t0 + tt < tokens ? to_float(x[(int64_t)(t0 + tt) * hidden + k]) : 0.f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.y * 8 + warp;
    if (e >= experts) return;
    const float* wr = router + (int64_t)e * hidden;
    float acc[RT];
#pragma unroll
    for (int tt = 0; tt < RT; ++tt) acc[tt] = 0.f;
#pragma unroll 4
    for (int k = lane; k < hidden; k += 32) {
        const float wv = __ldg(wr + k);
#pragma unroll
        for (int tt = 0; tt < RT; ++tt) acc[tt] = fmaf(x_s[tt * hidden + k], wv, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < RT; ++tt) {
        const float v = warp_sum(acc[tt]);
        if (lane == 0 && t0 + tt < tokens) logits[(int64_t)(t0 + tt) * experts + e] = v;
    }
}

// The choice of one token by one warp, from its logits. `work`: 4 * experts floats of shared
// memory (s[E], choice[E], group score[E], candidates[E]).
__device__ __forceinline__ void route_choose(const float* logits, const float* __restrict__ correction,
                                             int* __restrict__ chosen, float* __restrict__ weights,
                                             float* work, int lane, int64_t t, int experts, int top,
                                             int group_count, int group_keep, float route_scale) {
    float* s_s = work;
    float* choice_s = s_s + experts;
    float* group_s = choice_s + experts;
    float* cand_s = group_s + experts;
    for (int e = lane; e < experts; e += 32) {
        const float s = 1.f / (1.f + expf(-logits[e]));
        s_s[e] = s;
        choice_s[e] = s + correction[e];
        cand_s[e] = -INFINITY;
    }
    __syncwarp();
    const int size = experts / group_count;
    for (int g = lane; g < group_count; g += 32) {
        float first = -INFINITY, second = -INFINITY;
        for (int j = 0; j < size; ++j) {
            const float v = choice_s[g * size + j];
            if (v > first) {
                second = first;
                first = v;
            } else if (v > second) {
                second = v;
            }
        }
        group_s[g] = size >= 2 ? first + second : first;
    }
    __syncwarp();
    for (int round = 0; round < group_keep; ++round) {
        float v = -INFINITY;
        int i = -1;
        for (int g = lane; g < group_count; g += 32)
            if (group_s[g] > -INFINITY) take_better(v, i, group_s[g], g);
        warp_argmax(v, i);
        if (i < 0) break;                       // nothing comparable is left (a row of NaN)
        for (int j = lane; j < size; j += 32) cand_s[i * size + j] = choice_s[i * size + j];
        if (lane == 0) group_s[i] = -INFINITY;
        __syncwarp();
    }
    for (int round = 0; round < top; ++round) {
        float v = -INFINITY;
        int i = -1;
        for (int e = lane; e < experts; e += 32)
            if (cand_s[e] > -INFINITY) take_better(v, i, cand_s[e], e);
        warp_argmax(v, i);
        if (lane == 0) {
            // a row that is not a number chooses nothing: it gets an expert and no weight
            chosen[(int64_t)t * top + round] = i >= 0 ? i : round % experts;
            weights[(int64_t)t * top + round] = i >= 0 ? s_s[i] * route_scale : 0.f;
            if (i >= 0) cand_s[i] = -INFINITY;
        }
        __syncwarp();
    }
}

// A warp per token.
__global__ void route_select_kernel(const float* __restrict__ logits,
                                    const float* __restrict__ correction, int* __restrict__ chosen,
                                    float* __restrict__ weights, int tokens, int experts, int top,
                                    int group_count, int group_keep, float route_scale) {
    grid_dependency_sync();
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    route_choose(logits + (int64_t)t * experts, correction, chosen, weights,
                 sm + (size_t)warp * 4 * experts, lane, t, experts, top, group_count, group_keep,
                 route_scale);
}

// Few tokens (a decode step): logits and choice in one launch, a block of eight warps per
// token. The warps take the experts in turn (a lane its share of the expert's row), the
// logits meet in shared memory and the first warp chooses.
template <typename T>
__global__ void __launch_bounds__(256)
route_token_kernel(const T* __restrict__ x, const float* __restrict__ router,
                   const float* __restrict__ correction, int* __restrict__ chosen,
                   float* __restrict__ weights, int hidden, int experts, int top, int group_count,
                   int group_keep, float route_scale) {
    grid_dependency_sync();
    extern __shared__ float sm[];                  // x [hidden], logits [experts], work [4 experts]
    float* x_s = sm;
    float* logit_s = x_s + hidden;
    const int t = blockIdx.x;
    for (int k = threadIdx.x; k < hidden; k += blockDim.x) x_s[k] = to_float(x[(int64_t)t * hidden + k]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = warp; e < experts; e += 8) {
        const float* wr = router + (int64_t)e * hidden;
        float acc = 0.f;
#pragma unroll 4
        for (int k = lane; k < hidden; k += 32) acc = fmaf(x_s[k], __ldg(wr + k), acc);
        acc = warp_sum(acc);
        if (lane == 0) logit_s[e] = acc;
    }
    __syncthreads();
    if (warp == 0)
        route_choose(logit_s, correction, chosen, weights, logit_s + experts, lane, t, experts, top,
                     group_count, group_keep, route_scale);
}

// One block sorts the step's pairs by expert. plan: [0] tiles in all, then tile_expert[cap],
// tile_row0[cap], tile_rows[cap], then perm[pairs] (pair = token * top + choice, grouped by
// expert; the order inside an expert is arbitrary and changes no result), then ends[experts]
// (where each expert's rows end in the sorted order) and place[pairs] (the sorted row of
// every pair): what a library's grouped product and the sum behind it need.
__global__ void __launch_bounds__(1024)
expert_plan_kernel(const int* __restrict__ chosen, int pairs, int experts, int cap, int bm,
                   int* __restrict__ plan) {
    grid_dependency_sync();
    extern __shared__ int ism[];
    int* count_s = ism;                 // [experts]
    int* start_s = ism + experts;       // [experts]
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count_s[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < experts) atomicAdd(&count_s[e], 1);
    }
    __syncthreads();
    int* tile_expert = plan + 1;
    int* tile_row0 = tile_expert + cap;
    int* tile_rows = tile_row0 + cap;
    int* perm = tile_rows + cap;
    int* ends = perm + pairs;
    int* place = ends + experts;
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            start_s[e] = at;
            for (int r = 0; r < count_s[e] && tiles < cap; r += bm) {
                tile_expert[tiles] = e;
                tile_row0[tiles] = at + r;
                tile_rows[tiles] = min(bm, count_s[e] - r);
                ++tiles;
            }
            at += count_s[e];
            ends[e] = at;
        }
        plan[0] = tiles;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < experts) {
            const int at = atomicAdd(&start_s[e], 1);
            perm[at] = i;
            place[i] = at;
        }
    }
}

// sorted[i][:] = x[perm[i] / top][:]: the tokens' rows in the order of the plan, 16 bytes a
// thread (hidden a multiple of 8).
__global__ void expert_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ perm,
                                     __nv_bfloat16* __restrict__ sorted, int pairs, int top,
                                     int hidden, const float* __restrict__ row_scale) {
    grid_dependency_sync();
    const int chunks = hidden / 8;
    const int64_t total = (int64_t)pairs * chunks;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / chunks;
        const int c = (int)(i - r * chunks);
        const int t = perm[r] / top;
        uint4 piece = reinterpret_cast<const uint4*>(x + (int64_t)t * hidden)[c];
        if (row_scale != nullptr) {       // a weight on the expert's input: the row times it
            const float rs = row_scale[perm[r]];
            __nv_bfloat162* two = reinterpret_cast<__nv_bfloat162*>(&piece);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 v = __bfloat1622float2(two[j]);
                two[j] = __floats2bfloat162_rn(v.x * rs, v.y * rs);
            }
        }
        reinterpret_cast<uint4*>(sorted + r * hidden)[c] = piece;
    }
}

// out[t][n] = sum_j weights[t][j] * y[place[t * top + j]][n], j ascending: the weighted sum
// over rows that lie in the plan's order.
__global__ void expert_combine_sorted_kernel(const __nv_bfloat16* __restrict__ y,
                                             const int* __restrict__ place,
                                             const float* __restrict__ weights, float* __restrict__ out,
                                             int tokens, int top, int hidden) {
    grid_dependency_sync();
    const int64_t total = (int64_t)tokens * hidden;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / hidden;
        const int n = (int)(i - t * hidden);
        float acc = 0.f;
        for (int j = 0; j < top; ++j)
            acc = fmaf(weights != nullptr ? weights[t * top + j] : 1.f,
                       __bfloat162float(y[(int64_t)place[t * top + j] * hidden + n]), acc);
        out[i] = acc;
    }
}

// MODE 0: rows of x gathered by pair (token = pair / top) times [gate rows; up rows] of the
//         tile's expert, out = silu(gate) * up into act[sorted row][n] (type TA).
// MODE 1: act[sorted row] times the expert's down matrix, into y[pair][n] (float32).
// w: [experts][w_rows][K] with K contiguous (w_rows = 2 N in MODE 0, N in MODE 1).
template <typename TA, typename TW, int MODE>
__global__ void __launch_bounds__(256)
expert_product_kernel(const TA* __restrict__ a, int a_ld, const TW* __restrict__ w,
                      void* __restrict__ out, const int* __restrict__ plan, int cap, int top,
                      int K, int N, const float* __restrict__ row_scale) {
    grid_dependency_sync();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int* tile_expert = plan + 1;
    const int* tile_row0 = tile_expert + cap;
    const int* tile_rows = tile_row0 + cap;
    const int* perm = tile_rows + cap;
    const int e = tile_expert[tile], row0 = tile_row0[tile], rows = tile_rows[tile];
    const int n0 = blockIdx.y * EX_BN;
    constexpr int PARTS = MODE == 0 ? 2 : 1;
    __shared__ float a_s[EX_BK][EX_BM + 1];
    __shared__ __align__(16) float w_s[PARTS][EX_BK][EX_BN + 4];
    __shared__ int src_s[EX_BM];
    const int tid = threadIdx.x;
    if (tid < EX_BM) {
        int src = -1;
        if (tid < rows) src = MODE == 0 ? perm[row0 + tid] / top : row0 + tid;
        src_s[tid] = src;
    }
    __syncthreads();
    const int ty = tid >> 4, tx = tid & 15;
    float acc[PARTS][2][4];
#pragma unroll
    for (int p = 0; p < PARTS; ++p)
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[p][r][c] = 0.f;
    const int w_rows = PARTS * N;
    const TW* we = w + (int64_t)e * w_rows * K;
    const int ar = tid >> 3, ak = (tid & 7) * 4;          // this thread's piece of the A tile
    const int wn = tid >> 2, wk = (tid & 3) * 8;          // ... and of each W tile
    for (int k0 = 0; k0 < K; k0 += EX_BK) {
        {
            const int src = src_s[ar];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = k0 + ak + j;
                a_s[ak + j][ar] = (src >= 0 && k < K) ? to_float(a[(int64_t)src * a_ld + k]) : 0.f;
            }
        }
#pragma unroll
        for (int p = 0; p < PARTS; ++p) {
            const int n = n0 + wn;
            const TW* wrow = we + (int64_t)(p * N + n) * K;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int k = k0 + wk + j;
                w_s[p][wk + j][wn] = (n < N && k < K) ? to_float(wrow[k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < EX_BK; ++k) {
            const float a0 = a_s[k][ty * 2], a1 = a_s[k][ty * 2 + 1];
#pragma unroll
            for (int p = 0; p < PARTS; ++p) {
                const float4 wv = *reinterpret_cast<const float4*>(&w_s[p][k][tx * 4]);
                acc[p][0][0] = fmaf(a0, wv.x, acc[p][0][0]);
                acc[p][0][1] = fmaf(a0, wv.y, acc[p][0][1]);
                acc[p][0][2] = fmaf(a0, wv.z, acc[p][0][2]);
                acc[p][0][3] = fmaf(a0, wv.w, acc[p][0][3]);
                acc[p][1][0] = fmaf(a1, wv.x, acc[p][1][0]);
                acc[p][1][1] = fmaf(a1, wv.y, acc[p][1][1]);
                acc[p][1][2] = fmaf(a1, wv.z, acc[p][1][2]);
                acc[p][1][3] = fmaf(a1, wv.w, acc[p][1][3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int lr = ty * 2 + r;
        if (lr >= rows) continue;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int n = n0 + tx * 4 + c;
            if (n >= N) continue;
            if (MODE == 0) {
                // a weight on the expert's INPUT scales both products (they have no bias)
                const float rs = row_scale != nullptr ? row_scale[perm[row0 + lr]] : 1.f;
                const float g = acc[0][r][c] * rs, u = acc[PARTS - 1][r][c] * rs;
                reinterpret_cast<TA*>(out)[(int64_t)(row0 + lr) * N + n] =
                    from_float<TA>(g / (1.f + expf(-g)) * u);
            } else {
                reinterpret_cast<float*>(out)[(int64_t)perm[row0 + lr] * N + n] = acc[0][r][c];
            }
        }
    }
}


// ---- the same products on the tensor cores (bfloat16) --------------------------------------
// mma.sync m16n8k16 with float32 accumulators. A block of eight warps takes a tile of TC_BM
// rows of one expert and TC_BN output columns (in MODE 0 the TC_BN gate rows and the TC_BN up
// rows of the matrix that belong to them), K in rounds of TC_BK through three shared-memory
// stages filled by 16-byte cp.async (rows of 128 bytes, the 16-byte pieces of a row permuted
// by the row's low bits so that ldmatrix meets no bank twice). The warps lie 4 x 2: a warp
// owns 32 rows and 32 columns (of both parts), so a fragment of the matrix serves two row
// tiles. Rows beyond the tile, columns beyond N and pieces beyond K are filled with zeros by
// the copy itself. A row's sums do not depend on the other rows of its tile.
constexpr int TC_BM = 128, TC_BN = 64, TC_BK = 64, TC_STAGES = 3, TC_THREADS = 256;

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool full) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = full ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                 "{%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MODE>
__global__ void __launch_bounds__(TC_THREADS)
expert_product_mma_kernel(const __nv_bfloat16* __restrict__ a, int a_ld,
                          const __nv_bfloat16* __restrict__ w, void* __restrict__ out,
                          const int* __restrict__ plan, int cap, int top, int K, int N,
                          const float* __restrict__ row_scale) {
    grid_dependency_sync();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int* tile_expert = plan + 1;
    const int* tile_row0 = tile_expert + cap;
    const int* tile_rows = tile_row0 + cap;
    const int* perm = tile_rows + cap;
    const int e = tile_expert[tile], row0 = tile_row0[tile], rows = tile_rows[tile];
    const int n0 = blockIdx.y * TC_BN;
    constexpr int PARTS = MODE == 0 ? 2 : 1;
    constexpr int W_ROWS = PARTS * TC_BN;
    extern __shared__ __align__(128) unsigned char tc_smem[];
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(tc_smem);            // [stages][TC_BM][TC_BK]
    __nv_bfloat16* w_s = a_s + TC_STAGES * TC_BM * TC_BK;                       // [stages][W_ROWS][TC_BK]
    __shared__ int src_s[TC_BM];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wr = warp >> 1, wc = warp & 1;
    if (tid < TC_BM) {
        int src = -1;
        if (tid < rows) src = MODE == 0 ? perm[row0 + tid] / top : row0 + tid;
        src_s[tid] = src;
    }
    __syncthreads();
    const __nv_bfloat16* we = w + (int64_t)e * (PARTS * N) * K;
    const int rounds = (K + TC_BK - 1) / TC_BK;

    // every call commits a group, an empty one beyond the last round, so that the count of
    // groups in flight tells which round has landed
    auto fill = [&](int round) {
        if (round < rounds) {
            const int stage = round % TC_STAGES, k0 = round * TC_BK;
            for (int idx = tid; idx < TC_BM * 8; idx += TC_THREADS) {
                const int r = idx >> 3, c = idx & 7;
                const int src = src_s[r];
                const bool ok = src >= 0 && k0 + c * 8 < K;
                const __nv_bfloat16* from = ok ? a + (int64_t)src * a_ld + k0 + c * 8 : a;
                cp_async_16(a_s + (stage * TC_BM + r) * TC_BK + ((c ^ (r & 7)) * 8), from, ok);
            }
            for (int idx = tid; idx < W_ROWS * 8; idx += TC_THREADS) {
                const int r = idx >> 3, c = idx & 7;
                const int part = r / TC_BN, n = n0 + (r - part * TC_BN);
                const bool ok = n < N && k0 + c * 8 < K;
                const __nv_bfloat16* from = ok ? we + (int64_t)(part * N + n) * K + k0 + c * 8 : w;
                cp_async_16(w_s + (stage * W_ROWS + r) * TC_BK + ((c ^ (r & 7)) * 8), from, ok);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // acc[part][row tile of 16][column tile of 8][4]
    float acc[PARTS][2][4][4];
#pragma unroll
    for (int p = 0; p < PARTS; ++p)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[p][i][j][c] = 0.f;

#pragma unroll
    for (int st = 0; st < TC_STAGES - 1; ++st) fill(st);
    for (int kt = 0; kt < rounds; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(TC_STAGES - 2) : "memory");
        __syncthreads();        // round kt has landed for everyone, and round kt - 1 is consumed
        fill(kt + TC_STAGES - 1);
        const int stage = kt % TC_STAGES;
        const __nv_bfloat16* as = a_s + (stage * TC_BM + wr * 32) * TC_BK;
        const __nv_bfloat16* ws = w_s + stage * W_ROWS * TC_BK;
        // a decode step's tiles hold a handful of rows: a warp whose 32 rows are all beyond
        // the tile's has nothing to multiply (it still copies and meets the others)
        if (wr * 32 >= rows) continue;
        const bool second = wr * 32 + 16 < rows;
#pragma unroll
        for (int kk = 0; kk < TC_BK / 16; ++kk) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = i * 16 + (lane & 15), c = kk * 2 + (lane >> 4);
                if (i == 0 || second) ldmatrix_x4(af[i], as + r * TC_BK + ((c ^ (r & 7)) * 8));
            }
#pragma unroll
            for (int p = 0; p < PARTS; ++p) {
#pragma unroll
                for (int j2 = 0; j2 < 2; ++j2) {
                    // two column tiles of 8 at once: lanes 0-15 the first (its two k halves),
                    // lanes 16-31 the second
                    uint32_t bf[4];
                    const int r = p * TC_BN + wc * 32 + j2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                    const int c = kk * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(bf, ws + r * TC_BK + ((c ^ (r & 7)) * 8));
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        if (i == 1 && !second) continue;
                        mma_bf16_16816(acc[p][i][2 * j2], af[i], bf[0], bf[1]);
                        mma_bf16_16816(acc[p][i][2 * j2 + 1], af[i], bf[2], bf[3]);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int lr = wr * 32 + i * 16 + g + h * 8;
            if (lr >= rows) continue;
            const int64_t dst_row = MODE == 0 ? (int64_t)(row0 + lr) : (int64_t)perm[row0 + lr];
            const float rs = (MODE == 0 && row_scale != nullptr) ? row_scale[perm[row0 + lr]] : 1.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + wc * 32 + j * 8 + 2 * t4;
                if (n >= N) continue;
                const float v0 = acc[0][i][j][2 * h] * rs, v1 = acc[0][i][j][2 * h + 1] * rs;
                if (MODE == 0) {
                    const float u0 = acc[PARTS - 1][i][j][2 * h] * rs, u1 = acc[PARTS - 1][i][j][2 * h + 1] * rs;
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + dst_row * N + n;
                    const float r0 = v0 / (1.f + expf(-v0)) * u0, r1 = v1 / (1.f + expf(-v1)) * u1;
                    if (n + 1 < N && (N & 1) == 0)
                        *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(r0, r1);
                    else {
                        o[0] = __float2bfloat16_rn(r0);
                        if (n + 1 < N) o[1] = __float2bfloat16_rn(r1);
                    }
                } else {
                    float* o = reinterpret_cast<float*>(out) + dst_row * N + n;
                    if (n + 1 < N && (N & 1) == 0)
                        *reinterpret_cast<float2*>(o) = make_float2(v0, v1);
                    else {
                        o[0] = v0;
                        if (n + 1 < N) o[1] = v1;
                    }
                }
            }
        }
    }
}

template <int MODE>
int launch_expert_product_mma(const void* a, int a_ld, const void* w, void* out, const int* plan,
                              int cap, int top, int K, int N, const float* row_scale, cudaStream_t s) {
    constexpr int PARTS = MODE == 0 ? 2 : 1;
    const size_t smem = (size_t)TC_STAGES * (TC_BM + PARTS * TC_BN) * TC_BK * sizeof(__nv_bfloat16);
    // (with the kernel's static shared memory this is beyond the 48 KB a launch gets unasked)
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(expert_product_mma_kernel<MODE>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    dim3 grid(cap, (N + TC_BN - 1) / TC_BN);
    if (grid.y > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    MB_LAUNCH((expert_product_mma_kernel<MODE>), grid, TC_THREADS, smem, s, (const __nv_bfloat16*)a, a_ld,
              (const __nv_bfloat16*)w, out, plan, cap, top, K, N, row_scale);
    return launch_status();
}

// out[t][n] = sum_j weights[t][j] * y[t * top + j][n], j ascending (weights null: ones).
__global__ void expert_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights,
                                      float* __restrict__ out, int tokens, int top, int hidden) {
    grid_dependency_sync();
    const int64_t total = (int64_t)tokens * hidden;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / hidden;
        const int n = (int)(i - t * hidden);
        float acc = 0.f;
        for (int j = 0; j < top; ++j)
            acc = fmaf(weights != nullptr ? weights[t * top + j] : 1.f, y[(t * top + j) * hidden + n], acc);
        out[i] = acc;
    }
}

template <typename TA, typename TW>
int launch_expert_product(int mode, const void* a, int a_ld, const void* w, void* out,
                          const int* plan, int cap, int top, int K, int N, const float* row_scale,
                          cudaStream_t s) {
    dim3 grid(cap, (N + EX_BN - 1) / EX_BN);
    if (grid.y > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (mode == 0)
        MB_LAUNCH((expert_product_kernel<TA, TW, 0>), grid, 256, 0, s, (const TA*)a, a_ld, (const TW*)w,
                  out, plan, cap, top, K, N, row_scale);
    else
        MB_LAUNCH((expert_product_kernel<TA, TW, 1>), grid, 256, 0, s, (const TA*)a, a_ld, (const TW*)w,
                  out, plan, cap, top, K, N, row_scale);
    return launch_status();
}

}  // namespace mb

using namespace mb;

// x_dtype: the activations' type; router and correction are float32. `logits`: float32
// scratch of tokens * experts.
MB_EXPORT int mb_route_experts(const void* x, int x_dtype, const float* router,
                               const float* correction, float* logits, int* chosen, float* weights,
                               int tokens, int hidden, int experts, int top, int group_count,
                               int group_keep, float route_scale, void* stream) {
    if (tokens <= 0) return MB_OK;
    if (experts <= 0 || top <= 0 || top > experts || group_count <= 0 || experts % group_count ||
        group_keep <= 0 || group_keep > group_count)
        return MB_ERR_UNSUPPORTED_SIZE;
    int warps = 4;
    while (warps > 1 && (size_t)warps * 4 * experts * sizeof(float) > 40 * 1024) warps >>= 1;
    const size_t smem = (size_t)warps * 4 * experts * sizeof(float);
    if (smem > 40 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t one = (size_t)(hidden + 5 * experts) * sizeof(float);
    if (tokens <= 32 && one <= 48 * 1024) {
        if (x_dtype == MB_F32)
            MB_LAUNCH((route_token_kernel<float>), tokens, 256, one, s, (const float*)x, router, correction,
                      chosen, weights, hidden, experts, top, group_count, group_keep, route_scale);
        else if (x_dtype == MB_BF16)
            MB_LAUNCH((route_token_kernel<__nv_bfloat16>), tokens, 256, one, s, (const __nv_bfloat16*)x,
                      router, correction, chosen, weights, hidden, experts, top, group_count, group_keep,
                      route_scale);
        else
            return MB_ERR_BAD_DTYPE;
        return launch_status();
    }
    // many tokens: four a block, so that an expert's row is read once for four of them
    const bool many = tokens > 64 && (size_t)4 * hidden * sizeof(float) <= 48 * 1024;
    const int rt = many ? 4 : 1;
    const size_t x_smem = (size_t)rt * hidden * sizeof(float);
    if (x_smem > 48 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid((tokens + rt - 1) / rt, (experts + 7) / 8);
    if (grid.y > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    typedef __nv_bfloat16 bf;
    if (x_dtype == MB_F32) {
        if (many) MB_LAUNCH((router_logits_kernel<float, 4>), grid, 256, x_smem, s, (const float*)x, router, logits, tokens, hidden, experts);
        else MB_LAUNCH((router_logits_kernel<float, 1>), grid, 256, x_smem, s, (const float*)x, router, logits, tokens, hidden, experts);
    } else if (x_dtype == MB_BF16) {
        if (many) MB_LAUNCH((router_logits_kernel<bf, 4>), grid, 256, x_smem, s, (const bf*)x, router, logits, tokens, hidden, experts);
        else MB_LAUNCH((router_logits_kernel<bf, 1>), grid, 256, x_smem, s, (const bf*)x, router, logits, tokens, hidden, experts);
    } else {
        return MB_ERR_BAD_DTYPE;
    }
    if (cudaGetLastError() != cudaSuccess) return MB_ERR_LAUNCH;
    MB_LAUNCH((route_select_kernel), (tokens + warps - 1) / warps, warps * 32, smem, s, logits, correction,
              chosen, weights, tokens, experts, top, group_count, group_keep, route_scale);
    return launch_status();
}

// Rows per tile of the grouped products for this dtype and these sizes: the tensor-core
// kernel (bfloat16, K a multiple of 8 in both products) takes tiles of 128, the CUDA-core
// kernel tiles of 32.
MB_EXPORT int mb_expert_tile_rows(int dtype, int hidden, int ff) {
    return (dtype == MB_BF16 && hidden % 8 == 0 && ff % 8 == 0) ? TC_BM : EX_BM;
}

// The most tiles of `bm` rows a step of `pairs` pairs over `experts` experts can have.
MB_EXPORT int mb_expert_tile_cap(int pairs, int experts, int bm) {
    const int bound = pairs / bm + experts;
    return pairs < bound ? pairs : bound;
}

// Integers the plan needs: 1 + 3 * cap + 2 * pairs + experts.
MB_EXPORT int mb_expert_plan(const int* chosen, int pairs, int experts, int cap, int bm, int* plan,
                             void* stream) {
    if (pairs <= 0) return MB_OK;
    if (experts <= 0 || experts > 4096 || cap <= 0 || bm <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    MB_LAUNCH((expert_plan_kernel), 1, 1024, (size_t)2 * experts * sizeof(int), (cudaStream_t)stream,
              chosen, pairs, experts, cap, bm, plan);
    return launch_status();
}

// mode 0: gate/up with the SiLU gate (a = the tokens' rows, out = act in the activations'
// type); mode 1: down (a = act, out = float32 rows per pair). dtype: of a and w alike.
// `bm`: the tile height the plan was made with (mb_expert_tile_rows), which names the kernel.
MB_EXPORT int mb_expert_product(int mode, const void* a, int a_ld, const void* w, void* out,
                                const int* plan, int cap, int top, int K, int N, int dtype, int bm,
                                const float* row_scale, void* stream) {
    if (cap <= 0) return MB_OK;
    if (K <= 0 || N <= 0 || (mode != 0 && mode != 1)) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (bm == TC_BM) {
        if (dtype != MB_BF16 || K % 8 || a_ld % 8 || (((uintptr_t)a | (uintptr_t)w) & 15))
            return MB_ERR_ALIGNMENT;
        return mode == 0 ? launch_expert_product_mma<0>(a, a_ld, w, out, plan, cap, top, K, N, row_scale, s)
                         : launch_expert_product_mma<1>(a, a_ld, w, out, plan, cap, top, K, N, nullptr, s);
    }
    if (bm != EX_BM) return MB_ERR_UNSUPPORTED_SIZE;
    if (dtype == MB_F32)
        return launch_expert_product<float, float>(mode, a, a_ld, w, out, plan, cap, top, K, N, row_scale, s);
    if (dtype == MB_BF16)
        return launch_expert_product<__nv_bfloat16, __nv_bfloat16>(mode, a, a_ld, w, out, plan, cap, top,
                                                                   K, N, row_scale, s);
    return MB_ERR_BAD_DTYPE;
}

MB_EXPORT int mb_expert_gather(const void* x, const int* perm, void* sorted, int pairs, int top,
                               int hidden, const float* row_scale, void* stream) {
    if (pairs <= 0) return MB_OK;
    if (hidden % 8 || (((uintptr_t)x | (uintptr_t)sorted) & 15)) return MB_ERR_ALIGNMENT;
    const long long want = ((long long)pairs * (hidden / 8) + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    MB_LAUNCH((expert_gather_kernel), blocks, 256, 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, perm,
              (__nv_bfloat16*)sorted, pairs, top, hidden, row_scale);
    return launch_status();
}

MB_EXPORT int mb_expert_combine_sorted(const void* y, const int* place, const float* weights,
                                       float* out, int tokens, int top, int hidden, void* stream) {
    const long long total = (long long)tokens * hidden;
    if (total <= 0) return MB_OK;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    MB_LAUNCH((expert_combine_sorted_kernel), blocks, 256, 0, (cudaStream_t)stream,
              (const __nv_bfloat16*)y, place, weights, out, tokens, top, hidden);
    return launch_status();
}

MB_EXPORT int mb_expert_combine(const float* y, const float* weights, float* out, int tokens,
                                int top, int hidden, void* stream) {
    const long long total = (long long)tokens * hidden;
    if (total <= 0) return MB_OK;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    MB_LAUNCH((expert_combine_kernel), blocks, 256, 0, (cudaStream_t)stream, y, weights, out, tokens,
              top, hidden);
    return launch_status();
}
