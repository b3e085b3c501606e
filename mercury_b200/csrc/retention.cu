// Retention: linear attention with a fixed decay per head and neither softmax nor denominator.
// Per head, with q and k rotated by the token's position (the first rot_dim numbers of the
// head, halves or neighbours paired) and k then multiplied by key_scale:
//     S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,
// S a d x dv matrix that starts at zero and is carried from token to token in the request's
// state slot, in float32 like everything else here.
//
// A block takes one head of one sequence and 32 of its dv columns; a column is held by 8
// lanes, each with a run of ceil(d / 8) rows in registers (the state lies column by column,
// [head][column][row], so a lane's run is contiguous in memory). The step's tokens of the
// sequence are staged 16 at a time in shared memory, rotated and scaled on the way; per
// token a lane updates its rows and adds up its share of the read-out, and three shuffles
// finish the column's sum. The walk of a column is the same whatever else is in the batch
// and however the prompt was cut.
#include "common.cuh"

namespace mb {

constexpr int RT_TOKENS = 16;
constexpr int RT_COLS = 32;

template <int RMAX>
__global__ void __launch_bounds__(256)
retention_scan_kernel(const float* __restrict__ pre, int ld, int at_q, int at_k, int at_v,
                      const float* __restrict__ decay, float key_scale,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dim,
                      int interleaved, const int* __restrict__ positions, float* __restrict__ cells,
                      int64_t cell_stride, const int* __restrict__ q_start,
                      const int* __restrict__ slots, float* __restrict__ out, int heads, int d, int dv) {
    grid_dependency_sync();
    extern __shared__ float rt_smem[];
    float* q_s = rt_smem;                       // [RT_TOKENS][d]
    float* k_s = q_s + RT_TOKENS * d;           // [RT_TOKENS][d]
    float* v_s = k_s + RT_TOKENS * d;           // [RT_TOKENS][RT_COLS]
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * RT_COLS;
    const int begin = q_start[seq], end = q_start[seq + 1];
    if (end <= begin) return;
    const int tid = threadIdx.x, col = tid >> 3, sub = tid & 7;
    const int p = col0 + col;
    const int per = (d + 7) / 8;                // rows a lane holds
    const int r0 = sub * per;
    const float g = decay[head];
    float* cell = cells + (int64_t)slots[seq] * cell_stride + ((int64_t)head * dv + (p < dv ? p : 0)) * d;
    float S[RMAX];
#pragma unroll
    for (int i = 0; i < RMAX; ++i) S[i] = (i < per && r0 + i < d && p < dv) ? cell[r0 + i] : 0.f;
    const int pairs = rot_dim / 2;

    for (int t0 = begin; t0 < end; t0 += RT_TOKENS) {
        const int count = end - t0 < RT_TOKENS ? end - t0 : RT_TOKENS;
        __syncthreads();
        // q and k of the tile's tokens, rotated; k also scaled
        for (int idx = tid; idx < count * 2 * d; idx += blockDim.x) {
            const int tt = idx / (2 * d), rest = idx - tt * 2 * d;
            const int which = rest / d, c = rest - which * d;
            const float* x = pre + (int64_t)(t0 + tt) * ld + (which ? at_k : at_q) + head * d;
            float val;
            if (c < rot_dim) {
                int i, other;
                bool first;
                if (interleaved) {
                    i = c >> 1, first = !(c & 1), other = first ? c + 1 : c - 1;
                } else {
                    first = c < pairs, i = first ? c : c - pairs, other = first ? c + pairs : c - pairs;
                }
                const int pos = checked_position(positions[t0 + tt]);
                const float cs = cos_t[(int64_t)pos * pairs + i], sn = sin_t[(int64_t)pos * pairs + i];
                val = first ? x[c] * cs - x[other] * sn : x[c] * cs + x[other] * sn;
            } else {
                val = x[c];
            }
            (which ? k_s : q_s)[tt * d + c] = which ? val * key_scale : val;
        }
        for (int idx = tid; idx < count * RT_COLS; idx += blockDim.x) {
            const int tt = idx / RT_COLS, c = idx - tt * RT_COLS;
            v_s[idx] = col0 + c < dv ? pre[(int64_t)(t0 + tt) * ld + at_v + head * dv + col0 + c] : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < count; ++tt) {
            const float v = v_s[tt * RT_COLS + col];
            const float* kr = k_s + tt * d + r0;
            const float* qr = q_s + tt * d + r0;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < RMAX; ++i) {
                if (i < per && r0 + i < d) {
                    S[i] = fmaf(g, S[i], kr[i] * v);
                    o = fmaf(S[i], qr[i], o);
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (sub == 0 && p < dv) out[(int64_t)(t0 + tt) * heads * dv + head * dv + p] = o;
        }
    }
    if (p < dv) {
#pragma unroll
        for (int i = 0; i < RMAX; ++i)
            if (i < per && r0 + i < d) cell[r0 + i] = S[i];
    }
}

}  // namespace mb

using namespace mb;

// pre: [tokens][ld] float32 holding q (heads * d) at at_q, k at at_k and v (heads * dv) at at_v.
// cells: [slots][cell_stride] float32, a head's matrix column by column ([head][dv][d]).
// out: [tokens][heads * dv] float32. cos_t / sin_t: [positions][rot_dim / 2] (null: rot_dim 0).
MB_EXPORT int mb_retention_scan(const float* pre, int ld, int at_q, int at_k, int at_v,
                                const float* decay, float key_scale, const float* cos_t,
                                const float* sin_t, int rot_dim, int interleaved, const int* positions,
                                float* cells, long long cell_stride, const int* q_start,
                                const int* slots, float* out, int num_seqs, int heads, int d, int dv,
                                void* stream) {
    if (num_seqs <= 0) return MB_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || d > 256 || heads > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (rot_dim < 0 || (rot_dim & 1) || rot_dim > d || (rot_dim > 0 && (!cos_t || !sin_t)))
        return MB_ERR_UNSUPPORTED_SIZE;
    const int col_blocks = (dv + RT_COLS - 1) / RT_COLS;
    if (col_blocks > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid(num_seqs, heads, col_blocks);
    const size_t smem = (size_t)(2 * RT_TOKENS * d + RT_TOKENS * RT_COLS) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
#define MB_RT_CASE(R)                                                                              \
    MB_LAUNCH((retention_scan_kernel<R>), grid, 256, smem, s, pre, ld, at_q, at_k, at_v, decay,     \
              key_scale, cos_t, sin_t, rot_dim, interleaved, positions, cells, (int64_t)cell_stride, \
              q_start, slots, out, heads, d, dv)
    if (d <= 32) MB_RT_CASE(4);
    else if (d <= 64) MB_RT_CASE(8);
    else if (d <= 128) MB_RT_CASE(16);
    else MB_RT_CASE(32);
#undef MB_RT_CASE
    return launch_status();
}
