// Mixers whose memory is a matrix per head: a Mamba-2 state-space layer and a gated delta
// rule, with the short causal convolution in front of them and the gated group norm behind.
// A request's state lives in float32 in its slot: `cells` (the heads' matrices) and `tail`
// (the convolution's last taps - 1 inputs) are two regions of one state row, so both come
// as a pointer plus the distance between two slots' rows. Every kernel runs a step's tokens
// of sequence s (rows q_start[s] .. q_start[s+1]-1) in order from the state the step before
// left. Everything here is float32 in both engines; only the group norm's output (the input
// of the output projection) is stored in the activation type.
//
// Work split of the two scans: a block takes one head of one sequence (and a range of the
// head's columns p); inside a warp four columns are held by eight lanes each, lane `slice`
// keeping the matrix rows 4 (slice + 8 j) + {0, 1, 2, 3}, j = 0, 1, ..., of its column in
// registers: four neighbouring rows at a time, so that what a token brings for them comes
// out of shared memory as one 16-byte load (a warp's 32-bit loads of eight distinct words
// would use a quarter of the memory's width). A token's read-out is a sum over rows: four
// partial sums per lane, then three shuffles. The tokens' inputs are staged through shared
// memory thirty-two tokens at a time, so the block meets once per thirty-two tokens. A
// column's arithmetic is the same however the tokens were cut into steps.
//
// The template parameter S is the type the matrix is held in while a step runs. A float32
// matrix that takes in a thousand tokens one by one gathers a rounding error of some 1e-6 of
// its size, which is small beside bfloat16 activations and is what the bfloat16 engine runs
// with; the float32 engine holds the matrix and its sums in double inside a step (S =
// double) and rounds to float32 only when the step's last token is in, so a long prompt
// costs one rounding where it would cost one per token. The decay that multiplies the matrix
// at every token is computed in double in both and rounded once: an error of an ulp in expf
// that leans one way grows linearly with the number of tokens a contribution has to survive.
// Between steps the state is float32 in both.
#include "common.cuh"

namespace mb {

constexpr int SS_TILE = 32;      // tokens staged at a time
constexpr int SS_SLICES = 8;     // lanes that share a column

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float gate_f(float x, bool sigmoid) {
    return sigmoid ? 1.f / (1.f + expf(-x)) : silu_f(x);
}

// One float from global to shared memory without passing through registers (zeros when
// `take` is false), and the waits that go with it: the scans fetch the next tile of tokens
// while they walk the one before.
__device__ __forceinline__ void stage_float(float* dst, const float* src, bool take) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = take ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
// Four floats at once (both addresses 16-byte aligned).
__device__ __forceinline__ void stage_float4(float* dst, const float* src, bool take) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = take ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void stage_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void stage_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void stage_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// the matrix row that register i of lane `slice` holds
__device__ __forceinline__ int row_of(int slice, int i) { return 4 * (slice + SS_SLICES * (i >> 2)) + (i & 3); }

__device__ __forceinline__ float slice_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

__device__ __forceinline__ double softplus_f(double x) { return x > 40.0 ? x : log1p(exp(x)); }

__device__ __forceinline__ double slice_sum(double v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

// The same for a column shared by SL lanes (8, or the whole warp).
template <int SL>
__device__ __forceinline__ int row_in(int slice, int i) { return 4 * (slice + SL * (i >> 2)) + (i & 3); }

template <int SL, typename S>
__device__ __forceinline__ S lanes_sum(S v) {
#pragma unroll
    for (int o = 1; o < SL; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- short causal convolution --------------------------------------------------------------
// out[t][c] = act(sum_k w[c][k] * x[t - (taps - 1 - k)][c] + bias[c]), x = pre[:, offset + c]
// (row stride ld). Inputs from before the step come from the tail: tail[slot][(j - 1) *
// channels + c] is the input j tokens before the step's first token (zero before the
// sequence began, because a fresh slot is zeroed). The tail is not changed here.
__global__ void conv_act_kernel(const float* __restrict__ pre, int ld, int offset,
                                const float* __restrict__ w, const float* __restrict__ bias,
                                const float* __restrict__ tail, int64_t tail_stride,
                                const int* __restrict__ q_start, const int* __restrict__ slots,
                                const int* __restrict__ seq_of_token, float* __restrict__ out,
                                int channels, int taps, int act) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    const int seq = seq_of_token[t];
    if (c >= channels || seq < 0) return;
    const int begin = q_start[seq];
    const int at = t - begin;
    const float* past = tail + (int64_t)slots[seq] * tail_stride;
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) {
        const int src = at - (taps - 1 - k);
        const float x = src >= 0 ? pre[(int64_t)(begin + src) * ld + offset + c]
                                 : past[(int64_t)(-src - 1) * channels + c];
        acc = fmaf(w[c * taps + k], x, acc);
    }
    if (bias) acc += bias[c];
    if (act == 1) acc = silu_f(acc);
    out[(int64_t)t * channels + c] = acc;
}

// The tail after the step: the last taps - 1 inputs of (old tail, this step's inputs). Runs
// after every token's convolution has been taken.
__global__ void conv_tail_update_kernel(const float* __restrict__ pre, int ld, int offset,
                                        float* __restrict__ tail, int64_t tail_stride,
                                        const int* __restrict__ q_start,
                                        const int* __restrict__ slots, int channels, int taps) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], n = q_start[seq + 1] - begin;
    if (c >= channels || n <= 0) return;
    float* mine = tail + (int64_t)slots[seq] * tail_stride + c;
    float old[16];
    for (int j = 1; j < taps; ++j) old[j] = mine[(int64_t)(j - 1) * channels];
    for (int j = 1; j < taps; ++j) {
        const int idx = n - j;
        mine[(int64_t)(j - 1) * channels] =
            idx >= 0 ? pre[(int64_t)(begin + idx) * ld + offset + c] : old[j - n];
    }
}

// ---- Mamba-2 -------------------------------------------------------------------------------
// xbc: [tokens][inner + 2 * groups * n_state] = [x | B | C] behind convolution and SiLU;
// pre[:, dt_offset + head] the raw step sizes. Per head, with B and C of the head's group:
//   dt = softplus(raw + dt_bias);  S <- exp(neg_rate * dt) S + dt * B x^T;  y = S^T C + skip * x
// S is [n_state][vdim] at cells[slot][(head * n_state + n) * vdim + p].
//
// RUNS = false: a block walks all the step's tokens of its sequence from the state in `cells`.
// RUNS = true (long portions): the step's tokens of a sequence are cut into runs of `run_len`
// and block z walks run z from an EMPTY matrix: y gets the run's own part of the read-outs,
// `run_end` [sequence][run][head][n][p] the matrix the run ends with, `run_decay`
// [sequence][run][head] the product of its decays and `cum` [token][head] the product of the
// decays from the run's first token up to each token. Because the decay is one number per
// head, S_t = cum_t * S(run start) + (what the run itself added): mamba2_carry_kernel chains
// the runs' starts and mamba2_apply_kernel adds cum_t * C_t^T S(run start) to every y_t.
template <int NPT, typename S, bool RUNS>
__global__ void __launch_bounds__(512)
mamba2_scan_kernel(const float* __restrict__ xbc, const float* __restrict__ pre, int pre_ld,
                   int dt_offset, const float* __restrict__ dt_bias,
                   const float* __restrict__ neg_rate, const float* __restrict__ skip,
                   float* __restrict__ cells, int64_t cell_stride, const int* __restrict__ q_start,
                   const int* __restrict__ slots, float* __restrict__ y, int heads, int vdim,
                   int n_state, int groups, int chunks_per_head, int run_len,
                   float* __restrict__ run_end, float* __restrict__ run_decay,
                   float* __restrict__ cum) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float sm[];
    constexpr int NP = NPT * SS_SLICES;
    const int cols = (blockDim.x >> 5) * 4;
    // two stages of: B [SS_TILE][NP], C [SS_TILE][NP], x [SS_TILE][cols], raw step sizes [SS_TILE]
    const int stage_floats = 2 * SS_TILE * NP + SS_TILE * cols + SS_TILE;
    __shared__ S dt_s[SS_TILE], da_s[SS_TILE];
    const int head = blockIdx.x / chunks_per_head, chunk = blockIdx.x - head * chunks_per_head;
    const int seq = blockIdx.y;
    int begin = q_start[seq], end = q_start[seq + 1];
    if (RUNS) {
        begin += blockIdx.z * run_len;
        end = min(end, begin + run_len);
    }
    if (begin >= end) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slice = lane & 7, p_local = warp * 4 + (lane >> 3);
    const int p = chunk * cols + p_local;
    const bool live = p < vdim;
    const int inner = heads * vdim, width = inner + 2 * groups * n_state;
    const int g = head / (heads / groups);
    float* mine = RUNS ? run_end + (((int64_t)seq * gridDim.z + blockIdx.z) * heads + head) * n_state * vdim
                       : cells + (int64_t)slots[seq] * cell_stride + (int64_t)head * n_state * vdim;
    S s[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = row_of(slice, i);
        s[i] = (!RUNS && live && n < n_state) ? (S)mine[(int64_t)n * vdim + p] : (S)0;
    }
    const float rate = neg_rate[head], bias = dt_bias[head], d_skip = skip[head];
    __shared__ float run_cum;                 // product of the run's decays so far
    if (RUNS && tid == 0) run_cum = 1.f;
    auto fetch = [&](int stage, int t0) {
        float* b_to = sm + stage * stage_floats;
        float* c_to = b_to + SS_TILE * NP;
        float* x_to = c_to + SS_TILE * NP;
        float* raw_to = x_to + SS_TILE * cols;
        const int nt = min(SS_TILE, end - t0);
        for (int idx = tid; idx < nt * NP; idx += blockDim.x) {
            const int tt = idx / NP, n = idx - tt * NP;
            const float* row = xbc + (int64_t)(t0 + tt) * width + inner + g * n_state;
            const bool take = n < n_state;
            stage_float(b_to + idx, take ? row + n : xbc, take);
            stage_float(c_to + idx, take ? row + groups * n_state + n : xbc, take);
        }
        for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
            const int tt = idx / cols, pl = idx - tt * cols;
            const int pp = chunk * cols + pl;
            const bool take = pp < vdim;
            stage_float(x_to + idx, take ? xbc + (int64_t)(t0 + tt) * width + head * vdim + pp : xbc, take);
        }
        if (tid < nt) stage_float(raw_to + tid, pre + (int64_t)(t0 + tid) * pre_ld + dt_offset + head, true);
        stage_commit();
    };
    fetch(0, begin);
    int turn = 0;
    for (int t0 = begin; t0 < end; t0 += SS_TILE, turn ^= 1) {
        const int nt = min(SS_TILE, end - t0);
        const float* b_s = sm + turn * stage_floats;
        const float* c_s = b_s + SS_TILE * NP;
        const float* x_s = c_s + SS_TILE * NP;
        const float* raw_s = x_s + SS_TILE * cols;
        // the tile after this one is on its way while this one is walked (its stage was
        // left by everyone at the end of the turn before)
        if (t0 + SS_TILE < end) {
            fetch(turn ^ 1, t0 + SS_TILE);
            stage_wait_but_one();
        } else {
            stage_wait_all();
        }
        __syncthreads();
        if (tid < nt) {
            // in double whatever S is: a few numbers a tile, and the decay comes out rounded
            // to nearest instead of leaning one way
            const double dt = softplus_f((double)raw_s[tid] + (double)bias);
            dt_s[tid] = (S)dt;
            da_s[tid] = (S)exp((double)rate * dt);
        }
        __syncthreads();
        if (RUNS && tid == 0 && chunk == 0) {
            float c = run_cum;
            for (int tt = 0; tt < nt; ++tt) {
                c *= (float)da_s[tt];
                cum[(int64_t)(t0 + tt) * heads + head] = c;
            }
            run_cum = c;
        }
        for (int tt = 0; tt < nt; ++tt) {
            const float x = x_s[tt * cols + p_local];
            const S da = da_s[tt];
            const S dtx = dt_s[tt] * (S)x;
            const float4* bt = reinterpret_cast<const float4*>(b_s + tt * NP) + slice;
            const float4* ct = reinterpret_cast<const float4*>(c_s + tt * NP) + slice;
            S part[4] = {(S)0, (S)0, (S)0, (S)0};
#pragma unroll
            for (int j = 0; j < NPT / 4; ++j) {
                const float4 bv = bt[SS_SLICES * j], cv = ct[SS_SLICES * j];
                s[4 * j] = fma(da, s[4 * j], dtx * (S)bv.x);
                s[4 * j + 1] = fma(da, s[4 * j + 1], dtx * (S)bv.y);
                s[4 * j + 2] = fma(da, s[4 * j + 2], dtx * (S)bv.z);
                s[4 * j + 3] = fma(da, s[4 * j + 3], dtx * (S)bv.w);
                part[0] = fma(s[4 * j], (S)cv.x, part[0]);
                part[1] = fma(s[4 * j + 1], (S)cv.y, part[1]);
                part[2] = fma(s[4 * j + 2], (S)cv.z, part[2]);
                part[3] = fma(s[4 * j + 3], (S)cv.w, part[3]);
            }
            S acc = slice_sum((part[0] + part[1]) + (part[2] + part[3]));
            if (slice == 0 && live)
                y[(int64_t)(t0 + tt) * inner + head * vdim + p] = (float)fma((S)d_skip, (S)x, acc);
        }
        __syncthreads();                      // the stage may be refilled
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = row_of(slice, i);
        if (live && n < n_state) mine[(int64_t)n * vdim + p] = (float)s[i];
    }
    if (RUNS && tid == 0 && chunk == 0)
        run_decay[((int64_t)seq * gridDim.z + blockIdx.z) * heads + head] = run_cum;
}

// The runs' starts, one thread per element of a sequence's matrices: start(0) is the state
// the step found, start(r + 1) = decay(r) * start(r) + end(r); `run_end` is overwritten with
// the starts and the state becomes what follows the last run.
__global__ void mamba2_carry_kernel(float* __restrict__ run_end, const float* __restrict__ run_decay,
                                    float* __restrict__ cells, int64_t cell_stride,
                                    const int* __restrict__ q_start, const int* __restrict__ slots,
                                    int heads, int per_head, int run_len, int max_runs) {
    grid_dependency_sync();
    const int seq = blockIdx.y;
    const int n = q_start[seq + 1] - q_start[seq];
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (n <= 0 || e >= heads * per_head) return;
    const int head = e / per_head;
    const int runs = (n + run_len - 1) / run_len;
    float* cell = cells + (int64_t)slots[seq] * cell_stride + e;
    float carry = *cell;
    for (int r = 0; r < runs; ++r) {
        float* at = run_end + ((int64_t)seq * max_runs + r) * heads * per_head + e;
        const float ended = *at;
        *at = carry;
        carry = fmaf(run_decay[((int64_t)seq * max_runs + r) * heads + head], carry, ended);
    }
    *cell = carry;
}

// y_t += cum_t * C_t^T S(run start) for every token of every run: the same split of a head
// over lanes as the scan, the start held in registers, the tokens' C staged through shared
// memory.
template <int NPT>
__global__ void __launch_bounds__(512)
mamba2_apply_kernel(const float* __restrict__ xbc, const float* __restrict__ run_start,
                    const float* __restrict__ cum, const int* __restrict__ q_start,
                    float* __restrict__ y, int heads, int vdim, int n_state, int groups,
                    int chunks_per_head, int run_len) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float sm[];
    constexpr int NP = NPT * SS_SLICES;
    const int cols = (blockDim.x >> 5) * 4;
    const int stage_floats = SS_TILE * NP + SS_TILE;   // two stages of C [SS_TILE][NP], cum [SS_TILE]
    const int head = blockIdx.x / chunks_per_head, chunk = blockIdx.x - head * chunks_per_head;
    const int seq = blockIdx.y;
    const int begin = q_start[seq] + blockIdx.z * run_len;
    const int end = min(q_start[seq + 1], begin + run_len);
    if (begin >= end) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slice = lane & 7, p = chunk * cols + warp * 4 + (lane >> 3);
    const bool live = p < vdim;
    const int inner = heads * vdim, width = inner + 2 * groups * n_state;
    const int g = head / (heads / groups);
    const float* mine = run_start + (((int64_t)seq * gridDim.z + blockIdx.z) * heads + head) * n_state * vdim;
    float s[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = row_of(slice, i);
        s[i] = (live && n < n_state) ? mine[(int64_t)n * vdim + p] : 0.f;
    }
    auto fetch = [&](int stage, int t0) {
        float* c_to = sm + stage * stage_floats;
        float* cum_to = c_to + SS_TILE * NP;
        const int nt = min(SS_TILE, end - t0);
        for (int idx = tid; idx < nt * NP; idx += blockDim.x) {
            const int tt = idx / NP, n = idx - tt * NP;
            const bool take = n < n_state;
            stage_float(c_to + idx,
                        take ? xbc + (int64_t)(t0 + tt) * width + inner + (groups + g) * n_state + n : xbc, take);
        }
        if (tid < nt) stage_float(cum_to + tid, cum + (int64_t)(t0 + tid) * heads + head, true);
        stage_commit();
    };
    fetch(0, begin);
    int turn = 0;
    for (int t0 = begin; t0 < end; t0 += SS_TILE, turn ^= 1) {
        const int nt = min(SS_TILE, end - t0);
        const float* c_s = sm + turn * stage_floats;
        const float* cum_s = c_s + SS_TILE * NP;
        if (t0 + SS_TILE < end) {
            fetch(turn ^ 1, t0 + SS_TILE);
            stage_wait_but_one();
        } else {
            stage_wait_all();
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float4* ct = reinterpret_cast<const float4*>(c_s + tt * NP) + slice;
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < NPT / 4; ++j) {
                const float4 cv = ct[SS_SLICES * j];
                part[0] = fmaf(s[4 * j], cv.x, part[0]);
                part[1] = fmaf(s[4 * j + 1], cv.y, part[1]);
                part[2] = fmaf(s[4 * j + 2], cv.z, part[2]);
                part[3] = fmaf(s[4 * j + 3], cv.w, part[3]);
            }
            const float acc = slice_sum((part[0] + part[1]) + (part[2] + part[3]));
            if (slice == 0 && live) {
                float* at = y + (int64_t)(t0 + tt) * inner + head * vdim + p;
                *at = fmaf(cum_s[tt], acc, *at);
            }
        }
        __syncthreads();                      // the stage may be refilled
    }
}

// ---- gated delta rule ------------------------------------------------------------------------
// qkv: [tokens][2 * key_heads * dim + heads * vdim] = [q | k | v] behind convolution and SiLU;
// pre[:, beta_offset + head] and pre[:, decay_offset + head] the raw gate inputs. Head h
// reads q/k head h / (heads / key_heads). Per head:
//   q <- q / sqrt(sum q^2 + unit_eps) * dim^-1/2;  k <- k / sqrt(sum k^2 + unit_eps)
//   beta = sigmoid(raw_b);  g = exp(neg_rate * softplus(raw_a + dt_bias))
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// computed from the matrix as the token found it (A): S^T k = g A^T k and o = g A^T q +
// u (k . q), so one pass over a column's rows gives both sums. S is [dim][vdim] at
// cells[slot][(head * dim + d) * vdim + p].
// SL: the lanes that share a column, 8 as described above or 32 (one column a warp, four rows a
// lane at 128 rows): a quarter of the instructions per token and warp and four times the
// warps, for steps that bring too few (sequence, head) pairs to fill the machine otherwise.
template <int DPT, typename S, int SL = SS_SLICES>
__global__ void __launch_bounds__(512)
delta_rule_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ pre, int pre_ld,
                       int beta_offset, int decay_offset, const float* __restrict__ dt_bias,
                       const float* __restrict__ neg_rate, float unit_eps,
                       float* __restrict__ cells, int64_t cell_stride,
                       const int* __restrict__ q_start, const int* __restrict__ slots,
                       float* __restrict__ out, int heads, int key_heads, int dim, int vdim,
                       int chunks_per_head) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float sm[];
    constexpr int DP = DPT * SL;
    const int cols = (blockDim.x >> 5) * (32 / SL);
    // two stages of: q [SS_TILE][DP], k [SS_TILE][DP], v [SS_TILE][cols], raw beta and decay
    // inputs [2][SS_TILE]
    const int stage_floats = 2 * SS_TILE * DP + SS_TILE * cols + 2 * SS_TILE;
    __shared__ float beta_s[SS_TILE], kq_s[SS_TILE];
    __shared__ float kk_s[SS_TILE], kq_next_s[SS_TILE];   // k_t . k_(t+1) and k_t . q_(t+1), t even
    __shared__ S g_s[SS_TILE];
    // Two tokens per round where a lane's rows are few: both tokens' sums are taken against
    // the matrix as the first of them found it (A): with a_0 = A^T k_0 and a_1 = A^T k_1,
    //   u_0 = beta_0 (v_0 - g_0 a_0),   u_1 = beta_1 (v_1 - g_1 (g_0 a_1 + u_0 (k_0 . k_1)))
    // and the same for the read-outs, so that the sums over the lanes (the longest stretch of
    // a token's chain) are taken for two tokens side by side.
    constexpr bool PAIRS = DPT <= 8;
    const int head = blockIdx.x / chunks_per_head, chunk = blockIdx.x - head * chunks_per_head;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], end = q_start[seq + 1];
    if (begin >= end) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    const int slice = lane & (SL - 1), p_local = warp * (32 / SL) + lane / SL;
    const int p = chunk * cols + p_local;
    const bool live = p < vdim;
    const int qk = key_heads * dim, inner = heads * vdim, width = 2 * qk + inner;
    const int kh = head / (heads / key_heads);
    float* mine = cells + (int64_t)slots[seq] * cell_stride + (int64_t)head * dim * vdim;
    S s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = row_in<SL>(slice, i);
        s[i] = (live && d < dim) ? (S)mine[(int64_t)d * vdim + p] : (S)0;
    }
    const float rate = neg_rate[head], bias = dt_bias[head];
    const float q_scale = 1.f / sqrtf((float)dim);
    auto fetch = [&](int stage, int t0) {
        float* q_to = sm + stage * stage_floats;
        float* k_to = q_to + SS_TILE * DP;
        float* v_to = k_to + SS_TILE * DP;
        float* raw_to = v_to + SS_TILE * cols;
        const int nt = min(SS_TILE, end - t0);
        for (int idx = tid; idx < nt * DP; idx += blockDim.x) {
            const int tt = idx / DP, d = idx - tt * DP;
            const float* row = qkv + (int64_t)(t0 + tt) * width + kh * dim;
            const bool take = d < dim;
            stage_float(q_to + idx, take ? row + d : qkv, take);
            stage_float(k_to + idx, take ? row + qk + d : qkv, take);
        }
        for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
            const int tt = idx / cols, pl = idx - tt * cols;
            const int pp = chunk * cols + pl;
            const bool take = pp < vdim;
            stage_float(v_to + idx, take ? qkv + (int64_t)(t0 + tt) * width + 2 * qk + head * vdim + pp : qkv, take);
        }
        if (tid < nt) {
            const float* row = pre + (int64_t)(t0 + tid) * pre_ld;
            stage_float(raw_to + tid, row + beta_offset + head, true);
            stage_float(raw_to + SS_TILE + tid, row + decay_offset + head, true);
        }
        stage_commit();
    };
    fetch(0, begin);
    int turn = 0;
    for (int t0 = begin; t0 < end; t0 += SS_TILE, turn ^= 1) {
        const int nt = min(SS_TILE, end - t0);
        float* q_s = sm + turn * stage_floats;
        float* k_s = q_s + SS_TILE * DP;
        const float* v_s = k_s + SS_TILE * DP;
        const float* raw_s = v_s + SS_TILE * cols;
        if (t0 + SS_TILE < end) {
            fetch(turn ^ 1, t0 + SS_TILE);
            stage_wait_but_one();
        } else {
            stage_wait_all();
        }
        __syncthreads();
        if (tid < nt) {
            beta_s[tid] = 1.f / (1.f + expf(-raw_s[tid]));
            g_s[tid] = (S)exp((double)rate * softplus_f((double)raw_s[SS_TILE + tid] + (double)bias));
        }
        // unit vectors, and the token's k . q
        for (int tt = warp; tt < nt; tt += warps) {
            float qq = 0.f, kk = 0.f, cross = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const float a = q_s[tt * DP + d], b = k_s[tt * DP + d];
                qq = fmaf(a, a, qq);
                kk = fmaf(b, b, kk);
                cross = fmaf(a, b, cross);
            }
            qq = warp_sum(qq);
            kk = warp_sum(kk);
            cross = warp_sum(cross);
            const float rq = q_scale / sqrtf(qq + unit_eps), rk = 1.f / sqrtf(kk + unit_eps);
            for (int d = lane; d < dim; d += 32) {
                q_s[tt * DP + d] *= rq;
                k_s[tt * DP + d] *= rk;
            }
            if (lane == 0) kq_s[tt] = cross * rq * rk;
        }
        __syncthreads();
        int first_single = 0;
        if (PAIRS) {
            for (int tt = 2 * warp; tt + 1 < nt; tt += 2 * warps) {
                float kk = 0.f, kq = 0.f;
                for (int d = lane; d < dim; d += 32) {
                    const float k0 = k_s[tt * DP + d];
                    kk = fmaf(k0, k_s[(tt + 1) * DP + d], kk);
                    kq = fmaf(k0, q_s[(tt + 1) * DP + d], kq);
                }
                kk = warp_sum(kk);
                kq = warp_sum(kq);
                if (lane == 0) {
                    kk_s[tt] = kk;
                    kq_next_s[tt] = kq;
                }
            }
            __syncthreads();
            for (int tt = 0; tt + 1 < nt; tt += 2) {
                const float4* q0 = reinterpret_cast<const float4*>(q_s + tt * DP) + slice;
                const float4* k0 = reinterpret_cast<const float4*>(k_s + tt * DP) + slice;
                const float4* q1 = reinterpret_cast<const float4*>(q_s + (tt + 1) * DP) + slice;
                const float4* k1 = reinterpret_cast<const float4*>(k_s + (tt + 1) * DP) + slice;
                float4 k0v[DPT / 4], k1v[DPT / 4];
                S a0 = (S)0, a1 = (S)0, b0 = (S)0, b1 = (S)0;
#pragma unroll
                for (int j = 0; j < DPT / 4; ++j) {
                    k0v[j] = k0[SL * j];
                    k1v[j] = k1[SL * j];
                    const float4 q0v = q0[SL * j], q1v = q1[SL * j];
                    a0 += (s[4 * j] * (S)k0v[j].x + s[4 * j + 1] * (S)k0v[j].y) +
                          (s[4 * j + 2] * (S)k0v[j].z + s[4 * j + 3] * (S)k0v[j].w);
                    a1 += (s[4 * j] * (S)k1v[j].x + s[4 * j + 1] * (S)k1v[j].y) +
                          (s[4 * j + 2] * (S)k1v[j].z + s[4 * j + 3] * (S)k1v[j].w);
                    b0 += (s[4 * j] * (S)q0v.x + s[4 * j + 1] * (S)q0v.y) +
                          (s[4 * j + 2] * (S)q0v.z + s[4 * j + 3] * (S)q0v.w);
                    b1 += (s[4 * j] * (S)q1v.x + s[4 * j + 1] * (S)q1v.y) +
                          (s[4 * j + 2] * (S)q1v.z + s[4 * j + 3] * (S)q1v.w);
                }
#pragma unroll
                for (int o = 1; o < SL; o <<= 1) {         // four sums side by side
                    a0 += __shfl_xor_sync(0xffffffffu, a0, o);
                    a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                    b0 += __shfl_xor_sync(0xffffffffu, b0, o);
                    b1 += __shfl_xor_sync(0xffffffffu, b1, o);
                }
                const S g0 = g_s[tt], g1 = g_s[tt + 1];
                const S u0 = (S)beta_s[tt] * ((S)v_s[tt * cols + p_local] - g0 * a0);
                const S u1 = (S)beta_s[tt + 1] *
                             ((S)v_s[(tt + 1) * cols + p_local] - g1 * (g0 * a1 + u0 * (S)kk_s[tt]));
                const S both = g1 * g0, c0 = g1 * u0;
#pragma unroll
                for (int j = 0; j < DPT / 4; ++j) {
                    s[4 * j] = fma(both, s[4 * j], fma((S)k0v[j].x, c0, (S)k1v[j].x * u1));
                    s[4 * j + 1] = fma(both, s[4 * j + 1], fma((S)k0v[j].y, c0, (S)k1v[j].y * u1));
                    s[4 * j + 2] = fma(both, s[4 * j + 2], fma((S)k0v[j].z, c0, (S)k1v[j].z * u1));
                    s[4 * j + 3] = fma(both, s[4 * j + 3], fma((S)k0v[j].w, c0, (S)k1v[j].w * u1));
                }
                if (slice == 0 && live) {
                    float* at = out + (int64_t)(t0 + tt) * inner + head * vdim + p;
                    at[0] = (float)fma(u0, (S)kq_s[tt], g0 * b0);
                    at[inner] = (float)fma(u1, (S)kq_s[tt + 1], g1 * (g0 * b1 + u0 * (S)kq_next_s[tt]));
                }
            }
            first_single = nt & ~1;             // an odd tile leaves its last token
        }
        for (int tt = first_single; tt < nt; ++tt) {
            const float4* qt = reinterpret_cast<const float4*>(q_s + tt * DP) + slice;
            const float4* kt = reinterpret_cast<const float4*>(k_s + tt * DP) + slice;
            float4 kv[DPT / 4];
            S pa[4] = {(S)0, (S)0, (S)0, (S)0}, pb[4] = {(S)0, (S)0, (S)0, (S)0};
#pragma unroll
            for (int j = 0; j < DPT / 4; ++j) {
                kv[j] = kt[SL * j];
                const float4 qv = qt[SL * j];
                pa[0] = fma(s[4 * j], (S)kv[j].x, pa[0]);
                pa[1] = fma(s[4 * j + 1], (S)kv[j].y, pa[1]);
                pa[2] = fma(s[4 * j + 2], (S)kv[j].z, pa[2]);
                pa[3] = fma(s[4 * j + 3], (S)kv[j].w, pa[3]);
                pb[0] = fma(s[4 * j], (S)qv.x, pb[0]);
                pb[1] = fma(s[4 * j + 1], (S)qv.y, pb[1]);
                pb[2] = fma(s[4 * j + 2], (S)qv.z, pb[2]);
                pb[3] = fma(s[4 * j + 3], (S)qv.w, pb[3]);
            }
            const S a = lanes_sum<SL, S>((pa[0] + pa[1]) + (pa[2] + pa[3]));
            const S b = lanes_sum<SL, S>((pb[0] + pb[1]) + (pb[2] + pb[3]));
            const S g = g_s[tt];
            const S u = (S)beta_s[tt] * ((S)v_s[tt * cols + p_local] - g * a);
#pragma unroll
            for (int j = 0; j < DPT / 4; ++j) {
                s[4 * j] = fma(g, s[4 * j], (S)kv[j].x * u);
                s[4 * j + 1] = fma(g, s[4 * j + 1], (S)kv[j].y * u);
                s[4 * j + 2] = fma(g, s[4 * j + 2], (S)kv[j].z * u);
                s[4 * j + 3] = fma(g, s[4 * j + 3], (S)kv[j].w * u);
            }
            if (slice == 0 && live)
                out[(int64_t)(t0 + tt) * inner + head * vdim + p] = (float)fma(u, (S)kq_s[tt], g * b);
        }
        __syncthreads();                      // the stage may be refilled
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = row_in<SL>(slice, i);
        if (live && d < dim) mine[(int64_t)d * vdim + p] = (float)s[i];
    }
}

// ---- generalized delta rule --------------------------------------------------------------------
// pre: [tokens][ld] float32 with r, k (heads * dim each), v (heads * vdim) and the raw removal
// rates a (heads * dim) at the given column offsets; decay_in: [tokens][heads * dim] raw decay
// inputs. Per head, with u = k / sqrt(sum k^2 + unit_eps), a = sigmoid(raw a) and w = exp(-
// decay_scale * sigmoid(raw decay)) per key channel:
//   S <- diag(w) S - (a * u) (u^T S) + k v^T,   o = S^T r,
// both terms reading the matrix as the token found it (A). Column p of S needs two sums over
// A's rows, x = u . A[:, p] and y = (w * r) . A[:, p]; then S[:, p] = w * A[:, p] - (a * u) x + k
// v_p and o_p = y - x ((a * u) . r) + v_p (k . r): one pass over the column per token. S is
// [dim][vdim] at cells[slot][(head * dim + d) * vdim + p]. The split of a head over lanes is the
// one described at the top of this file (eight lanes a column, four neighbouring rows at a
// time). With the matrices in double the decay is computed in double and rounded once.
template <int DPT, typename S, int TILE>
__global__ void __launch_bounds__(512)
general_delta_scan_kernel(const float* __restrict__ pre, int ld, int at_r, int at_k, int at_v, int at_a,
                          const float* __restrict__ decay_in, float decay_scale, float unit_eps,
                          float* __restrict__ cells, int64_t cell_stride,
                          const int* __restrict__ q_start, const int* __restrict__ slots,
                          float* __restrict__ out, int heads, int dim, int vdim, int chunks_per_head,
                          int vec4) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float sm[];
    constexpr int SL = SS_SLICES;
    constexpr int DP = DPT * SL;
    const int cols = (blockDim.x >> 5) * (32 / SL);
    // two stages of [r, then w * r | k | raw a, then a * u | raw decay, then w | v], filled by
    // cp.async a tile ahead, and the unit keys of the tile being walked
    const int stage_floats = 4 * TILE * DP + TILE * cols;
    float* u_s = sm + 2 * stage_floats;        // [TILE][DP]
    __shared__ float aur_s[TILE], kr_s[TILE];
    const int head = blockIdx.x / chunks_per_head, chunk = blockIdx.x - head * chunks_per_head;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], end = q_start[seq + 1];
    if (begin >= end) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    const int slice = lane & (SL - 1), p_local = warp * (32 / SL) + lane / SL;
    const int p = chunk * cols + p_local;
    const bool live = p < vdim;
    const int inner = heads * vdim;
    float* mine = cells + (int64_t)slots[seq] * cell_stride + (int64_t)head * dim * vdim;
    S s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = row_in<SL>(slice, i);
        s[i] = (live && d < dim) ? (S)mine[(int64_t)d * vdim + p] : (S)0;
    }
    auto fetch = [&](int stage, int t0) {
        float* r_to = sm + stage * stage_floats;
        float* k_to = r_to + TILE * DP;
        float* a_to = k_to + TILE * DP;
        float* w_to = a_to + TILE * DP;
        float* v_to = w_to + TILE * DP;
        const int nt = min(TILE, end - t0);
        if (vec4) {
            // every row, offset and size a multiple of four floats: 16 bytes a copy
            for (int idx = tid; idx < nt * (DP / 4); idx += blockDim.x) {
                const int tt = idx / (DP / 4), d = 4 * (idx - tt * (DP / 4));
                const bool take = d < dim;
                const float* row = pre + (int64_t)(t0 + tt) * ld + head * dim + d;
                stage_float4(r_to + 4 * idx, take ? row + at_r : pre, take);
                stage_float4(k_to + 4 * idx, take ? row + at_k : pre, take);
                stage_float4(a_to + 4 * idx, take ? row + at_a : pre, take);
                stage_float4(w_to + 4 * idx,
                             take ? decay_in + (int64_t)(t0 + tt) * heads * dim + head * dim + d : pre, take);
            }
            for (int idx = tid; idx < nt * (cols / 4); idx += blockDim.x) {
                const int tt = idx / (cols / 4), pp = chunk * cols + 4 * (idx - tt * (cols / 4));
                const bool take = pp < vdim;
                stage_float4(v_to + 4 * idx,
                             take ? pre + (int64_t)(t0 + tt) * ld + at_v + head * vdim + pp : pre, take);
            }
            stage_commit();
            return;
        }
        for (int idx = tid; idx < nt * DP; idx += blockDim.x) {
            const int tt = idx / DP, d = idx - tt * DP;
            const bool take = d < dim;
            const float* row = pre + (int64_t)(t0 + tt) * ld + head * dim + d;
            stage_float(r_to + idx, take ? row + at_r : pre, take);
            stage_float(k_to + idx, take ? row + at_k : pre, take);
            stage_float(a_to + idx, take ? row + at_a : pre, take);
            stage_float(w_to + idx, take ? decay_in + (int64_t)(t0 + tt) * heads * dim + head * dim + d : pre,
                        take);
        }
        for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
            const int tt = idx / cols, pp = chunk * cols + (idx - tt * cols);
            const bool take = pp < vdim;
            stage_float(v_to + idx, take ? pre + (int64_t)(t0 + tt) * ld + at_v + head * vdim + pp : pre, take);
        }
        stage_commit();
    };
    fetch(0, begin);
    int turn = 0;
    for (int t0 = begin; t0 < end; t0 += TILE, turn ^= 1) {
        const int nt = min(TILE, end - t0);
        float* wr_s = sm + turn * stage_floats;    // r, then w * r    [TILE][DP]
        float* k_s = wr_s + TILE * DP;             // k
        float* au_s = k_s + TILE * DP;             // raw a, then a * u
        float* w_s = au_s + TILE * DP;             // raw decay, then w
        const float* v_s = w_s + TILE * DP;        // [TILE][cols]
        if (t0 + TILE < end) {
            fetch(turn ^ 1, t0 + TILE);
            stage_wait_but_one();
        } else {
            stage_wait_all();
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += warps) {
            float kk = 0.f;
            for (int d = lane; d < dim; d += 32) kk = fmaf(k_s[tt * DP + d], k_s[tt * DP + d], kk);
            kk = warp_sum(kk);
            const float rk = 1.f / sqrtf(kk + unit_eps);
            float aur = 0.f, kr = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const int at = tt * DP + d;
                const float r = wr_s[at], k = k_s[at];
                const float u = k * rk;
                const float a = 1.f / (1.f + expf(-au_s[at]));
                // held in double, the matrices are owed a decay rounded once; beside bfloat16
                // activations float arithmetic serves (a dependent chain of double-precision
                // exponentials per tile was most of this kernel's time)
                float w;
                if constexpr (sizeof(S) == 8)
                    w = (float)exp(-(double)decay_scale / (1.0 + exp(-(double)w_s[at])));
                else
                    w = expf(-decay_scale / (1.f + expf(-w_s[at])));
                u_s[at] = u;
                au_s[at] = a * u;
                w_s[at] = w;
                wr_s[at] = w * r;
                aur = fmaf(a * u, r, aur);
                kr = fmaf(k, r, kr);
            }
            aur = warp_sum(aur);
            kr = warp_sum(kr);
            if (lane == 0) {
                aur_s[tt] = aur;
                kr_s[tt] = kr;
            }
            // rows beyond dim were staged as zeros and stay so, so padded rows of S stay zero
            for (int d = dim + lane; d < DP; d += 32) u_s[tt * DP + d] = 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float4* ut = reinterpret_cast<const float4*>(u_s + tt * DP) + slice;
            const float4* yt = reinterpret_cast<const float4*>(wr_s + tt * DP) + slice;
            S px[4] = {(S)0, (S)0, (S)0, (S)0}, py[4] = {(S)0, (S)0, (S)0, (S)0};
#pragma unroll
            for (int j = 0; j < DPT / 4; ++j) {
                const float4 uv = ut[SL * j], yv = yt[SL * j];
                px[0] = fma(s[4 * j], (S)uv.x, px[0]);
                px[1] = fma(s[4 * j + 1], (S)uv.y, px[1]);
                px[2] = fma(s[4 * j + 2], (S)uv.z, px[2]);
                px[3] = fma(s[4 * j + 3], (S)uv.w, px[3]);
                py[0] = fma(s[4 * j], (S)yv.x, py[0]);
                py[1] = fma(s[4 * j + 1], (S)yv.y, py[1]);
                py[2] = fma(s[4 * j + 2], (S)yv.z, py[2]);
                py[3] = fma(s[4 * j + 3], (S)yv.w, py[3]);
            }
            const S x = lanes_sum<SL, S>((px[0] + px[1]) + (px[2] + px[3]));
            const S y = lanes_sum<SL, S>((py[0] + py[1]) + (py[2] + py[3]));
            const S vp = (S)v_s[tt * cols + p_local];
            const float4* wt = reinterpret_cast<const float4*>(w_s + tt * DP) + slice;
            const float4* at = reinterpret_cast<const float4*>(au_s + tt * DP) + slice;
            const float4* kt = reinterpret_cast<const float4*>(k_s + tt * DP) + slice;
#pragma unroll
            for (int j = 0; j < DPT / 4; ++j) {
                const float4 wv = wt[SL * j], av = at[SL * j], kv = kt[SL * j];
                s[4 * j] = fma((S)wv.x, s[4 * j], fma((S)kv.x, vp, -(S)av.x * x));
                s[4 * j + 1] = fma((S)wv.y, s[4 * j + 1], fma((S)kv.y, vp, -(S)av.y * x));
                s[4 * j + 2] = fma((S)wv.z, s[4 * j + 2], fma((S)kv.z, vp, -(S)av.z * x));
                s[4 * j + 3] = fma((S)wv.w, s[4 * j + 3], fma((S)kv.w, vp, -(S)av.w * x));
            }
            if (slice == 0 && live)
                out[(int64_t)(t0 + tt) * inner + head * vdim + p] =
                    (float)(y - x * (S)aur_s[tt] + vp * (S)kr_s[tt]);
        }
        __syncthreads();                      // the stage may be refilled, the unit keys rewritten
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = row_in<SL>(slice, i);
        if (live && d < dim) mine[(int64_t)d * vdim + p] = (float)s[i];
    }
}

// out[t][c] = tanh(pre[t][offset + c]), float32.
__global__ void tanh_slice_kernel(const float* __restrict__ pre, int ld, int offset, int count,
                                  float* __restrict__ out, int64_t total) {
    grid_dependency_sync();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / count;
        out[i] = tanhf(pre[t * ld + offset + (i - t * count)]);
    }
}

// ---- gated group norm ------------------------------------------------------------------------
// y: [tokens][width] float32 in `groups` equal parts; gate = silu(pre[:, gate_offset + c]), or
// sigmoid(.) when bit 1 of `gate_first` is set. Bit 0 of gate_first: out = rmsnorm_part(y * gate)
// * w;  else: out = rmsnorm_part(y) * w * gate.
// w has `wn` entries and is read at c % wn (one weight per feature, or one per feature of a
// part, shared by the parts). A warp per (token, part).
template <typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ pre,
                                        int pre_ld, int gate_offset, const float* __restrict__ w,
                                        int wn, int groups, int size, float eps, int gate_first,
                                        TO* __restrict__ out, int tokens) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const int64_t id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (id >= (int64_t)tokens * groups) return;
    const int t = (int)(id / groups), part = (int)(id - (int64_t)t * groups);
    const int width = groups * size;
    const float* yr = y + (int64_t)t * width + part * size;
    const float* gr = pre + (int64_t)t * pre_ld + gate_offset + part * size;
    const bool first = gate_first & 1, sig = gate_first & 2;
    float ss = 0.f;
    for (int c = lane; c < size; c += 32) {
        float x = yr[c];
        if (first) x *= gate_f(gr[c], sig);
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)size + eps);
    TO* orow = out + (int64_t)t * width + part * size;
    for (int c = lane; c < size; c += 32) {
        const float gate = gate_f(gr[c], sig);
        float x = yr[c];
        if (first) x *= gate;
        x = x * rstd * w[(part * size + c) % wn];
        if (!first) x *= gate;
        orow[c] = from_float<TO>(x);
    }
}

// The same with a block of 128 threads per (token, part), for parts of 256 features and more
// (a warp alone would walk them in a long chain of dependent loads).
template <typename TO>
__global__ void __launch_bounds__(128)
gated_group_norm_block_kernel(const float* __restrict__ y, const float* __restrict__ pre, int pre_ld,
                              int gate_offset, const float* __restrict__ w, int wn, int groups,
                              int size, float eps, int gate_first, TO* __restrict__ out) {
    grid_dependency_sync();
    __shared__ float scratch[33];
    const int t = blockIdx.x / groups, part = blockIdx.x - t * groups;
    const int width = groups * size;
    const float* yr = y + (int64_t)t * width + part * size;
    const float* gr = pre + (int64_t)t * pre_ld + gate_offset + part * size;
    const bool first = gate_first & 1, sig = gate_first & 2;
    float ss = 0.f;
    for (int c = threadIdx.x; c < size; c += blockDim.x) {
        float x = yr[c];
        if (first) x *= gate_f(gr[c], sig);
        ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(ss / (float)size + eps);
    TO* orow = out + (int64_t)t * width + part * size;
    for (int c = threadIdx.x; c < size; c += blockDim.x) {
        const float gate = gate_f(gr[c], sig);
        float x = yr[c];
        if (first) x *= gate;
        x = x * rstd * w[(part * size + c) % wn];
        if (!first) x *= gate;
        orow[c] = from_float<TO>(x);
    }
}

// A step of few tokens per sequence (decoding): one thread per (sequence, channel) takes the
// convolution of the step's tokens in turn and then brings the tail up to date, in one launch.
__global__ void conv_act_update_kernel(const float* __restrict__ pre, int ld, int offset,
                                       const float* __restrict__ w, const float* __restrict__ bias,
                                       float* __restrict__ tail, int64_t tail_stride,
                                       const int* __restrict__ q_start, const int* __restrict__ slots,
                                       float* __restrict__ out, int channels, int taps, int act) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], n = q_start[seq + 1] - begin;
    if (c >= channels || n <= 0) return;
    float* mine = tail + (int64_t)slots[seq] * tail_stride + c;
    // hist[j]: the input j tokens before the token in hand (hist[0] the token itself)
    float hist[16], wk[16];
    for (int j = 1; j < taps; ++j) hist[j] = mine[(int64_t)(j - 1) * channels];
    for (int k = 0; k < taps; ++k) wk[k] = w[c * taps + k];
    const float b = bias ? bias[c] : 0.f;
    for (int t = 0; t < n; ++t) {
        hist[0] = pre[(int64_t)(begin + t) * ld + offset + c];
        float acc = 0.f;
        for (int k = 0; k < taps; ++k) acc = fmaf(wk[k], hist[taps - 1 - k], acc);
        if (bias) acc += b;
        if (act == 1) acc = silu_f(acc);
        out[(int64_t)(begin + t) * channels + c] = acc;
        for (int j = taps - 1; j >= 1; --j) hist[j] = hist[j - 1];
    }
    for (int j = 1; j < taps; ++j) mine[(int64_t)(j - 1) * channels] = hist[j];
}

}  // namespace mb

using namespace mb;

// The convolution of every token of the step and the tail's update behind it: one launch for
// steps of at most 8 tokens a sequence, two otherwise.
MB_EXPORT int mb_conv_act_update(const float* pre, int ld, int offset, const float* w,
                                 const float* bias, float* tail, long long tail_stride,
                                 const int* q_start, const int* slots, const int* seq_of_token,
                                 float* out, int tokens, int num_seqs, int max_q_len, int channels,
                                 int taps, int act, void* stream);

MB_EXPORT int mb_conv_act(const float* pre, int ld, int offset, const float* w, const float* bias,
                          const float* tail, long long tail_stride, const int* q_start,
                          const int* slots, const int* seq_of_token, float* out, int tokens,
                          int channels, int taps, int act, void* stream) {
    if (tokens <= 0 || channels <= 0) return MB_OK;
    if (taps < 1 || taps > 16 || tokens > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid((channels + 127) / 128, tokens);
    MB_LAUNCH((conv_act_kernel), grid, 128, 0, (cudaStream_t)stream, pre, ld, offset, w, bias, tail,
              (int64_t)tail_stride, q_start, slots, seq_of_token, out, channels, taps, act);
    return launch_status();
}

MB_EXPORT int mb_conv_tail_update(const float* pre, int ld, int offset, float* tail,
                                  long long tail_stride, const int* q_start, const int* slots,
                                  int num_seqs, int channels, int taps, void* stream) {
    if (num_seqs <= 0 || channels <= 0 || taps <= 1) return MB_OK;
    if (taps > 16 || num_seqs > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid((channels + 127) / 128, num_seqs);
    MB_LAUNCH((conv_tail_update_kernel), grid, 128, 0, (cudaStream_t)stream, pre, ld, offset, tail,
              (int64_t)tail_stride, q_start, slots, channels, taps);
    return launch_status();
}

MB_EXPORT int mb_conv_act_update(const float* pre, int ld, int offset, const float* w,
                                 const float* bias, float* tail, long long tail_stride,
                                 const int* q_start, const int* slots, const int* seq_of_token,
                                 float* out, int tokens, int num_seqs, int max_q_len, int channels,
                                 int taps, int act, void* stream) {
    if (tokens <= 0 || channels <= 0 || num_seqs <= 0) return MB_OK;
    if (taps < 1 || taps > 16 || num_seqs > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (max_q_len > 8) {
        const int rc = mb_conv_act(pre, ld, offset, w, bias, tail, tail_stride, q_start, slots,
                                   seq_of_token, out, tokens, channels, taps, act, stream);
        if (rc != MB_OK) return rc;
        return mb_conv_tail_update(pre, ld, offset, tail, tail_stride, q_start, slots, num_seqs,
                                   channels, taps, stream);
    }
    dim3 grid((channels + 127) / 128, num_seqs);
    MB_LAUNCH((conv_act_update_kernel), grid, 128, 0, (cudaStream_t)stream, pre, ld, offset, w, bias,
              tail, (int64_t)tail_stride, q_start, slots, out, channels, taps, act);
    return launch_status();
}

// Warps of a scan block (each holds four columns) and the blocks a head is cut into. A
// token costs a warp the same chain of instructions however many warps share its block, so
// while the blocks are fewer than two to an SM a head is cut into more of them (down to four
// warps, sixteen columns; fewer warps would spend longer staging a tile's inputs than
// walking it): the inputs are then staged once per block instead of once per head.
static void scan_shape(int vdim, int heads, int num_seqs, int* warps, int* chunks) {
    int w = (vdim + 3) / 4;
    if (w > 16) w = 16;
    while (w > 4 && (long long)heads * ((vdim + 4 * w - 1) / (4 * w)) * num_seqs < 2 * 148) w = (w + 1) / 2;
    *warps = w;
    *chunks = (vdim + 4 * w - 1) / (4 * w);
}

// A launch that wants more than 48 KB of dynamic shared memory has to say so first (wide
// matrices only: 256 rows).
template <typename K>
static bool allow_smem(K kernel, size_t smem) {
    // a kernel's static arrays count toward the 48 KB that need no opt-in: leave them room
    return smem + 2048 <= 48 * 1024 ||
           cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
}

// Tokens per run when long portions are cut into runs, and the floats of scratch that takes.
constexpr int SS_RUN = 128;

MB_EXPORT long long mb_mamba2_scratch_floats(int tokens, int num_seqs, int max_q_len, int heads,
                                            int vdim, int n_state) {
    const long long runs = (max_q_len + SS_RUN - 1) / SS_RUN;
    return (long long)num_seqs * runs * heads * ((long long)n_state * vdim + 1) + (long long)tokens * heads;
}

// `scratch`: null, or mb_mamba2_scratch_floats() floats: with it (and not `precise`) portions
// of 4 * SS_RUN tokens and more are cut into runs that blocks walk side by side.
MB_EXPORT int mb_mamba2_scan(const float* xbc, const float* pre, int pre_ld, int dt_offset,
                             const float* dt_bias, const float* neg_rate, const float* skip,
                             float* cells, long long cell_stride, const int* q_start,
                             const int* slots, float* y, int tokens, int num_seqs, int max_q_len,
                             int heads, int vdim, int n_state, int groups, int precise,
                             float* scratch, void* stream) {
    if (num_seqs <= 0) return MB_OK;
    if (heads <= 0 || vdim <= 0 || n_state <= 0 || n_state > 256 || groups <= 0 || heads % groups ||
        num_seqs > 65535)
        return MB_ERR_UNSUPPORTED_SIZE;
    const bool in_runs = scratch != nullptr && !precise && max_q_len >= 4 * SS_RUN;
    const int max_runs = in_runs ? (max_q_len + SS_RUN - 1) / SS_RUN : 1;
    if (max_runs > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    int warps, chunks;
    scan_shape(vdim, heads, num_seqs * max_runs, &warps, &chunks);
    dim3 grid(heads * chunks, num_seqs, max_runs);
    cudaStream_t s = (cudaStream_t)stream;
    const int per_head = n_state * vdim;
    float* run_end = scratch;
    float* run_decay = in_runs ? run_end + (int64_t)num_seqs * max_runs * heads * per_head : nullptr;
    float* cum = in_runs ? run_decay + (int64_t)num_seqs * max_runs * heads : nullptr;
#define MB_M2_ARGS xbc, pre, pre_ld, dt_offset, dt_bias, neg_rate, skip, cells, (int64_t)cell_stride, \
                   q_start, slots, y, heads, vdim, n_state, groups, chunks, SS_RUN, run_end, run_decay, cum
#define MB_M2_CASE(NPT)                                                                            \
    do {                                                                                           \
        const size_t smem = (size_t)2 * (2 * SS_TILE * NPT * SS_SLICES + SS_TILE * warps * 4 +      \
                                         SS_TILE) * sizeof(float);                                 \
        if (!allow_smem(mamba2_scan_kernel<NPT, double, false>, smem) ||                           \
            !allow_smem(mamba2_scan_kernel<NPT, float, false>, smem) ||                            \
            !allow_smem(mamba2_scan_kernel<NPT, float, true>, smem))                               \
            return MB_ERR_UNSUPPORTED_SIZE;                                                        \
        if (precise)                                                                               \
            MB_LAUNCH((mamba2_scan_kernel<NPT, double, false>), grid, warps * 32, smem, s, MB_M2_ARGS); \
        else if (!in_runs)                                                                         \
            MB_LAUNCH((mamba2_scan_kernel<NPT, float, false>), grid, warps * 32, smem, s, MB_M2_ARGS);  \
        else {                                                                                     \
            MB_LAUNCH((mamba2_scan_kernel<NPT, float, true>), grid, warps * 32, smem, s, MB_M2_ARGS);   \
            dim3 cgrid((heads * per_head + 255) / 256, num_seqs);                                  \
            MB_LAUNCH((mamba2_carry_kernel), cgrid, 256, 0, s, run_end, run_decay, cells,          \
                      (int64_t)cell_stride, q_start, slots, heads, per_head, SS_RUN, max_runs);    \
            const size_t asmem = (size_t)2 * (SS_TILE * NPT * SS_SLICES + SS_TILE) * sizeof(float); \
            if (!allow_smem(mamba2_apply_kernel<NPT>, asmem)) return MB_ERR_UNSUPPORTED_SIZE;      \
            MB_LAUNCH((mamba2_apply_kernel<NPT>), grid, warps * 32, asmem, s, xbc, run_end, cum,   \
                      q_start, y, heads, vdim, n_state, groups, chunks, SS_RUN);                   \
        }                                                                                          \
    } while (0)
    if (n_state <= 32) MB_M2_CASE(4);
    else if (n_state <= 64) MB_M2_CASE(8);
    else if (n_state <= 128) MB_M2_CASE(16);
    else MB_M2_CASE(32);
#undef MB_M2_CASE
#undef MB_M2_ARGS
    (void)tokens;
    return launch_status();
}

MB_EXPORT int mb_delta_rule_scan(const float* qkv, const float* pre, int pre_ld, int beta_offset,
                                 int decay_offset, const float* dt_bias, const float* neg_rate,
                                 float unit_eps, float* cells, long long cell_stride,
                                 const int* q_start, const int* slots, float* out, int num_seqs,
                                 int heads, int key_heads, int dim, int vdim, int precise,
                                 void* stream) {
    if (num_seqs <= 0) return MB_OK;
    if (heads <= 0 || key_heads <= 0 || heads % key_heads || dim <= 0 || dim > 256 || vdim <= 0 ||
        num_seqs > 65535)
        return MB_ERR_UNSUPPORTED_SIZE;
    int warps, chunks;
    scan_shape(vdim, heads, num_seqs, &warps, &chunks);
    dim3 grid(heads * chunks, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define MB_DR_CASE(DPT)                                                                            \
    do {                                                                                           \
        const size_t smem = (size_t)2 * (2 * SS_TILE * DPT * SS_SLICES + SS_TILE * warps * 4 +      \
                                         2 * SS_TILE) * sizeof(float);                             \
        if (!allow_smem(delta_rule_scan_kernel<DPT, double>, smem) ||                              \
            !allow_smem(delta_rule_scan_kernel<DPT, float>, smem))                                 \
            return MB_ERR_UNSUPPORTED_SIZE;                                                        \
        if (precise)                                                                               \
            MB_LAUNCH((delta_rule_scan_kernel<DPT, double>), grid, warps * 32, smem, s, qkv, pre,  \
                      pre_ld, beta_offset, decay_offset, dt_bias, neg_rate, unit_eps, cells,       \
                      (int64_t)cell_stride, q_start, slots, out, heads, key_heads, dim, vdim,      \
                      chunks);                                                                     \
        else                                                                                       \
            MB_LAUNCH((delta_rule_scan_kernel<DPT, float>), grid, warps * 32, smem, s, qkv, pre,   \
                      pre_ld, beta_offset, decay_offset, dt_bias, neg_rate, unit_eps, cells,       \
                      (int64_t)cell_stride, q_start, slots, out, heads, key_heads, dim, vdim,      \
                      chunks);                                                                     \
    } while (0)
    // few (sequence, head) pairs and matrices of 128 rows or 256: a column per warp
    if (!precise && dim > 64 && (long long)heads * ((vdim + 4 * warps - 1) / (4 * warps)) * num_seqs < 148) {
        const int wide_warps = vdim < 8 ? vdim : 8;
        const int wide_chunks = (vdim + wide_warps - 1) / wide_warps;
        dim3 wide_grid(heads * wide_chunks, num_seqs);
#define MB_DR_WIDE(DPT)                                                                            \
    do {                                                                                           \
        const size_t smem = (size_t)2 * (2 * SS_TILE * DPT * 32 + SS_TILE * wide_warps +           \
                                         2 * SS_TILE) * sizeof(float);                             \
        if (!allow_smem(delta_rule_scan_kernel<DPT, float, 32>, smem)) return MB_ERR_UNSUPPORTED_SIZE; \
        MB_LAUNCH((delta_rule_scan_kernel<DPT, float, 32>), wide_grid, wide_warps * 32, smem, s, qkv, \
                  pre, pre_ld, beta_offset, decay_offset, dt_bias, neg_rate, unit_eps, cells,      \
                  (int64_t)cell_stride, q_start, slots, out, heads, key_heads, dim, vdim,          \
                  wide_chunks);                                                                    \
    } while (0)
        if (dim <= 128) MB_DR_WIDE(4);
        else MB_DR_WIDE(8);
#undef MB_DR_WIDE
        return launch_status();
    }
    if (dim <= 32) MB_DR_CASE(4);
    else if (dim <= 64) MB_DR_CASE(8);
    else if (dim <= 128) MB_DR_CASE(16);
    else MB_DR_CASE(32);
#undef MB_DR_CASE
    return launch_status();
}

// The generalized delta rule over a step's tokens; `precise`: the matrices are held in double
// while the step runs. Key sizes up to 256.
MB_EXPORT int mb_general_delta_scan(const float* pre, int ld, int at_r, int at_k, int at_v, int at_a,
                                    const float* decay_in, float decay_scale, float unit_eps,
                                    float* cells, long long cell_stride, const int* q_start,
                                    const int* slots, float* out, int num_seqs, int heads, int dim,
                                    int vdim, int precise, void* stream) {
    if (num_seqs <= 0 || heads <= 0) return MB_OK;
    if (dim <= 0 || dim > 256 || vdim <= 0 || num_seqs > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    int warps = (vdim + 3) / 4;
    if (warps < 4) warps = 4;
    if (warps > 16) warps = 16;
    // a step of few sequences: narrower blocks over more of the device (a column's walk is
    // the same whichever block holds it, so the result does not depend on the split)
    while (warps > 8 && (long long)heads * num_seqs * ((vdim + warps * 4 - 1) / (warps * 4)) < 148)
        warps /= 2;
    const int vec4 = ld % 4 == 0 && at_r % 4 == 0 && at_k % 4 == 0 && at_v % 4 == 0 && at_a % 4 == 0 &&
                     dim % 4 == 0 && vdim % 4 == 0 && ((uintptr_t)pre & 15) == 0 &&
                     ((uintptr_t)decay_in & 15) == 0;
    const int cols = warps * 4;
    const int chunks = (vdim + cols - 1) / cols;
    dim3 grid(heads * chunks, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define MB_GD_CASE(DPT, TILE)                                                                      \
    do {                                                                                           \
        const size_t smem = (size_t)(9 * TILE * DPT * SS_SLICES + 2 * TILE * cols) * sizeof(float); \
        if (!allow_smem(general_delta_scan_kernel<DPT, double, TILE>, smem) ||                     \
            !allow_smem(general_delta_scan_kernel<DPT, float, TILE>, smem))                        \
            return MB_ERR_UNSUPPORTED_SIZE;                                                        \
        if (precise)                                                                               \
            MB_LAUNCH((general_delta_scan_kernel<DPT, double, TILE>), grid, warps * 32, smem, s, pre, \
                      ld, at_r, at_k, at_v, at_a, decay_in, decay_scale, unit_eps, cells,          \
                      (int64_t)cell_stride, q_start, slots, out, heads, dim, vdim, chunks, vec4);  \
        else                                                                                       \
            MB_LAUNCH((general_delta_scan_kernel<DPT, float, TILE>), grid, warps * 32, smem, s, pre, \
                      ld, at_r, at_k, at_v, at_a, decay_in, decay_scale, unit_eps, cells,          \
                      (int64_t)cell_stride, q_start, slots, out, heads, dim, vdim, chunks, vec4);  \
    } while (0)
    // (the widest matrices stage 16 tokens at a time: two stages of 32 would not fit)
    if (dim <= 32) MB_GD_CASE(4, 32);
    else if (dim <= 64) MB_GD_CASE(8, 32);
    else if (dim <= 128) MB_GD_CASE(16, 32);
    else MB_GD_CASE(32, 16);
#undef MB_GD_CASE
    return launch_status();
}

MB_EXPORT int mb_tanh_slice(const float* pre, int ld, int offset, int count, float* out, int tokens,
                            void* stream) {
    const long long total = (long long)tokens * count;
    if (total <= 0) return MB_OK;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    MB_LAUNCH((tanh_slice_kernel), blocks, 256, 0, (cudaStream_t)stream, pre, ld, offset, count, out,
              (int64_t)total);
    return launch_status();
}

// out_dtype: MB_F32 or MB_BF16.
MB_EXPORT int mb_gated_group_norm(const float* y, const float* pre, int pre_ld, int gate_offset,
                                  const float* w, int wn, int groups, int size, float eps,
                                  int gate_first, void* out, int out_dtype, int tokens,
                                  void* stream) {
    if (tokens <= 0) return MB_OK;
    if (groups <= 0 || size <= 0 || wn <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    const long long warps = (long long)tokens * groups;
    const long long blocks = (warps + 7) / 8;
    if (warps > 0x7fffffffLL) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (size >= 256) {
        if (out_dtype == MB_F32)
            MB_LAUNCH((gated_group_norm_block_kernel<float>), (int)warps, 128, 0, s, y, pre, pre_ld,
                      gate_offset, w, wn, groups, size, eps, gate_first, (float*)out);
        else if (out_dtype == MB_BF16)
            MB_LAUNCH((gated_group_norm_block_kernel<__nv_bfloat16>), (int)warps, 128, 0, s, y, pre,
                      pre_ld, gate_offset, w, wn, groups, size, eps, gate_first, (__nv_bfloat16*)out);
        else
            return MB_ERR_BAD_DTYPE;
        return launch_status();
    }
    if (out_dtype == MB_F32)
        MB_LAUNCH((gated_group_norm_kernel<float>), (int)blocks, 256, 0, s, y, pre, pre_ld, gate_offset,
                  w, wn, groups, size, eps, gate_first, (float*)out, tokens);
    else if (out_dtype == MB_BF16)
        MB_LAUNCH((gated_group_norm_kernel<__nv_bfloat16>), (int)blocks, 256, 0, s, y, pre, pre_ld,
                  gate_offset, w, wn, groups, size, eps, gate_first, (__nv_bfloat16*)out, tokens);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}
