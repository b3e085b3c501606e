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
// sequence are staged 32 at a time (16 for key sizes above 128) by asynchronous copies a tile
// ahead of the walk, with the rows of the rotation tables they need, and rotated and scaled
// in shared memory; per token a lane updates its rows and adds up its share of the read-out,
// and three shuffles finish the column's sum. The walk of a column is the same whatever else is in the batch
// and however the prompt was cut.
#include "common.cuh"

namespace mb {

constexpr int RT_COLS = 32;

__device__ __forceinline__ void rt_copy4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void rt_copy16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}

// One staged tile of `tt_max` tokens: q and k as projected [tt][d] each, v [tt][RT_COLS], and the
// tokens' cosines and sines [tt][pairs] each.
// RMAX: the rows a lane can hold; EXACT: d is 8 * RMAX (a lane's run is full and starts on a
// 16-byte boundary), so the walk needs no bounds and reads q and k four numbers at a time.
template <int RMAX, bool EXACT>
__global__ void __launch_bounds__(256)
retention_scan_kernel(const float* __restrict__ pre, int ld, int at_q, int at_k, int at_v,
                      const float* __restrict__ decay, float key_scale,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dim,
                      int interleaved, const int* __restrict__ positions, float* __restrict__ cells,
                      int64_t cell_stride, const int* __restrict__ q_start,
                      const int* __restrict__ slots, float* __restrict__ out, int heads, int d, int dv,
                      int tt_max, int wide) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float rt_smem[];
    const int pairs = rot_dim / 2;
    const int tile_floats = tt_max * (2 * d + RT_COLS + 2 * pairs);
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

    // a tile's rows are brought by asynchronous copies a tile ahead of the walk, 16 bytes a copy
    // where every offset allows (`wide`), else 4: a thread owns a token of the tile (8 or 16
    // threads a token) and strides over its numbers
    const int lanes_per_token = 256 / tt_max;           // 8 (32 tokens a tile) or 16
    const int my_tt = tid / lanes_per_token, my_l = tid - my_tt * lanes_per_token;
    auto issue = [&](int t0, float* buf) {
        const int count = end - t0 < tt_max ? end - t0 : tt_max;
        if (my_tt < count) {
            const int t = t0 + my_tt;
            const float* row = pre + (int64_t)t * ld;
            float* q_b = buf + my_tt * d;
            float* k_b = buf + tt_max * d + my_tt * d;
            float* v_b = buf + 2 * tt_max * d + my_tt * RT_COLS;
            float* c_b = buf + tt_max * (2 * d + RT_COLS) + my_tt * pairs;
            float* s_b = c_b + tt_max * pairs;
            const int64_t pos = pairs > 0 ? checked_position(positions[t]) : 0;
            if (wide) {
                for (int c = my_l * 4; c < d; c += lanes_per_token * 4) {
                    rt_copy16(q_b + c, row + at_q + head * d + c);
                    rt_copy16(k_b + c, row + at_k + head * d + c);
                }
                for (int c = my_l * 4; c < RT_COLS; c += lanes_per_token * 4)
                    if (col0 + c < dv) rt_copy16(v_b + c, row + at_v + head * dv + col0 + c);
                for (int i = my_l * 4; i < pairs; i += lanes_per_token * 4) {
                    rt_copy16(c_b + i, cos_t + pos * pairs + i);
                    rt_copy16(s_b + i, sin_t + pos * pairs + i);
                }
            } else {
                for (int c = my_l; c < d; c += lanes_per_token) {
                    rt_copy4(q_b + c, row + at_q + head * d + c);
                    rt_copy4(k_b + c, row + at_k + head * d + c);
                }
                for (int c = my_l; c < RT_COLS; c += lanes_per_token)
                    if (col0 + c < dv) rt_copy4(v_b + c, row + at_v + head * dv + col0 + c);
                for (int i = my_l; i < pairs; i += lanes_per_token) {
                    rt_copy4(c_b + i, cos_t + pos * pairs + i);
                    rt_copy4(s_b + i, sin_t + pos * pairs + i);
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    issue(begin, rt_smem);
    int turn = 0;
    for (int t0 = begin; t0 < end; t0 += tt_max, turn ^= 1) {
        const int count = end - t0 < tt_max ? end - t0 : tt_max;
        float* buf = rt_smem + turn * tile_floats;
        if (t0 + tt_max < end) {
            issue(t0 + tt_max, rt_smem + (turn ^ 1) * tile_floats);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        float* q_s = buf;
        float* k_s = buf + tt_max * d;
        const float* v_s = buf + 2 * tt_max * d;
        // in place: the rotation of q and k (a thread takes whole pairs), then the keys' scale
        if (my_tt < count) {
            const float* c_b = buf + tt_max * (2 * d + RT_COLS) + my_tt * pairs;
            const float* s_b = c_b + tt_max * pairs;
            for (int i = my_l; i < pairs; i += lanes_per_token) {
                const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + pairs;
                const float cs = c_b[i], sn = s_b[i];
                float* qr = q_s + my_tt * d;
                float* kr = k_s + my_tt * d;
                const float qa = qr[a], qb = qr[b], ka = kr[a], kb = kr[b];
                qr[a] = qa * cs - qb * sn;
                qr[b] = qb * cs + qa * sn;
                kr[a] = (ka * cs - kb * sn) * key_scale;
                kr[b] = (kb * cs + ka * sn) * key_scale;
            }
            for (int c = rot_dim + my_l; c < d; c += lanes_per_token) k_s[my_tt * d + c] *= key_scale;
        }
        __syncthreads();
#pragma unroll 4
        for (int tt = 0; tt < count; ++tt) {
            const float v = p < dv ? v_s[tt * RT_COLS + col] : 0.f;
            const float* kr = k_s + tt * d + r0;
            const float* qr = q_s + tt * d + r0;
            float o = 0.f;
            if (EXACT) {
                float o2 = 0.f;          // two partial sums: half as long a chain of additions
#pragma unroll
                for (int i = 0; i < RMAX; i += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
                    const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
                    S[i] = fmaf(g, S[i], k4.x * v);
                    S[i + 1] = fmaf(g, S[i + 1], k4.y * v);
                    S[i + 2] = fmaf(g, S[i + 2], k4.z * v);
                    S[i + 3] = fmaf(g, S[i + 3], k4.w * v);
                    o = fmaf(S[i], q4.x, o);
                    o2 = fmaf(S[i + 1], q4.y, o2);
                    o = fmaf(S[i + 2], q4.z, o);
                    o2 = fmaf(S[i + 3], q4.w, o2);
                }
                o += o2;
            } else {
#pragma unroll
                for (int i = 0; i < RMAX; ++i) {
                    if (i < per && r0 + i < d) {
                        S[i] = fmaf(g, S[i], kr[i] * v);
                        o = fmaf(S[i], qr[i], o);
                    }
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (sub == 0 && p < dv) out[(int64_t)(t0 + tt) * heads * dv + head * dv + p] = o;
        }
        __syncthreads();      // the tile is free for the copies of the tile after next
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
    // two tiles of 32 tokens (16 for key sizes above 128) in shared memory
    const int tt_max = d <= 128 ? 32 : 16;
    const size_t smem = (size_t)2 * tt_max * (2 * d + RT_COLS + rot_dim) * sizeof(float);
    // 16-byte copies need every row piece to start on a 16-byte boundary
    const int pairs = rot_dim / 2;
    const int wide = (d % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && at_q % 4 == 0 && at_k % 4 == 0 &&
                      at_v % 4 == 0 && pairs % 4 == 0 && ((uintptr_t)pre & 15) == 0 &&
                      (pairs == 0 || ((((uintptr_t)cos_t) | ((uintptr_t)sin_t)) & 15) == 0))
                         ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
#define MB_RT_CASE(R)                                                                              \
    do {                                                                                           \
        static size_t raised = 0;                                                                  \
        if (smem > 40 * 1024 && smem > raised) {                                                   \
            if (cudaFuncSetAttribute(retention_scan_kernel<R, true>,                               \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=    \
                    cudaSuccess ||                                                                 \
                cudaFuncSetAttribute(retention_scan_kernel<R, false>,                              \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=    \
                    cudaSuccess)                                                                   \
                return MB_ERR_UNSUPPORTED_SIZE;                                                    \
            raised = smem;                                                                         \
        }                                                                                          \
        if (d == 8 * R)                                                                            \
            MB_LAUNCH((retention_scan_kernel<R, true>), grid, 256, smem, s, pre, ld, at_q, at_k, at_v, \
                      decay, key_scale, cos_t, sin_t, rot_dim, interleaved, positions, cells,      \
                      (int64_t)cell_stride, q_start, slots, out, heads, d, dv, tt_max, wide);            \
        else                                                                                       \
            MB_LAUNCH((retention_scan_kernel<R, false>), grid, 256, smem, s, pre, ld, at_q, at_k, at_v, \
                      decay, key_scale, cos_t, sin_t, rot_dim, interleaved, positions, cells,      \
                      (int64_t)cell_stride, q_start, slots, out, heads, d, dv, tt_max, wide);            \
    } while (0)
    if (d <= 32) MB_RT_CASE(4);
    else if (d <= 64) MB_RT_CASE(8);
    else if (d <= 128) MB_RT_CASE(16);
    else MB_RT_CASE(32);
#undef MB_RT_CASE
    return launch_status();
}
