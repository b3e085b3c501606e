// Attention over a cached latent: what stands around the attention kernel itself.
//
// The cache keeps one row c of `rank` numbers per token. A head's key is Wuk_h c and its
// value Wuv_h c, so q_h . k_h = (Wuk_h^T q_h) . c: the query is taken into the latent space
// once per token (`head_linear` with the transposed up-projection), the attention kernel
// then runs all heads over the cached rows as one shared key/value head of size `rank`, and
// `head_linear` applies Wuv_h to each head's weighted sum of rows.
#include "common.cuh"

namespace mb {

// c = x / sqrt(mean(x^2) + eps) * w for x = pre[t][offset .. offset + rank), stored into the
// token's slot of the pages [page][1][slot][rank]. A warp per token; float32 arithmetic.
template <typename T>
__global__ void latent_norm_store_kernel(const float* __restrict__ pre, int ld, int offset,
                                         const void* __restrict__ w, int w_dtype, float eps,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token,
                                         const int* __restrict__ table, int max_pages,
                                         T* __restrict__ pages, int rank, int page_size,
                                         int tokens) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int pos = positions[t];
    const int page = table_page(table, seq, max_pages, pos / page_size);
    if (page < 0) return;
    const float* x = pre + (int64_t)t * ld + offset;
    float ss = 0.f;
    for (int c = lane; c < rank; c += 32) ss = fmaf(x[c], x[c], ss);
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)rank + eps);
    T* row = pages + ((int64_t)page * page_size + (pos % page_size)) * rank;
    for (int c = lane; c < rank; c += 32)
        row[c] = from_float<T>(x[c] * rstd * load_as_float(w, c, w_dtype));
}

// out[t][h][o] = sum_i w[h][i][o] * x[t][offset + h * in + i]: one small matrix per head, held
// input-major so that consecutive threads (outputs o) read consecutive addresses. A block
// computes 128 outputs of one head for HL_TOKENS tokens, the inputs staged token-minor; i
// ascends, so the order of each sum is fixed. Sums are float32.
template <typename TX, typename TW, typename TO, int HL_TOKENS>
__global__ void __launch_bounds__(128)
head_linear_kernel(const TX* __restrict__ x, int ld, int offset, const TW* __restrict__ w,
                   TO* __restrict__ out, int tokens, int heads, int in, int outs) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float x_s[];          // [in][HL_TOKENS]
    const int per = (outs + 127) / 128;
    const int otile = blockIdx.x % per;
    const int h = blockIdx.x / per;
    const int t0 = blockIdx.y * HL_TOKENS;
    for (int idx = threadIdx.x; idx < HL_TOKENS * in; idx += blockDim.x) {
        const int tt = idx / in, i = idx - tt * in;
        x_s[i * HL_TOKENS + tt] =
            t0 + tt < tokens ? to_float(x[(int64_t)(t0 + tt) * ld + offset + h * in + i]) : 0.f;
    }
    __syncthreads();
    const int o = otile * 128 + threadIdx.x;
    if (o >= outs) return;
    const TW* wh = w + (int64_t)h * in * outs + o;
    float acc[HL_TOKENS];
#pragma unroll
    for (int tt = 0; tt < HL_TOKENS; ++tt) acc[tt] = 0.f;
#pragma unroll 16
    for (int i = 0; i < in; ++i) {
        const float v = to_float(wh[(int64_t)i * outs]);
        const float4* row = reinterpret_cast<const float4*>(x_s + i * HL_TOKENS);
#pragma unroll
        for (int q = 0; q < HL_TOKENS / 4; ++q) {
            const float4 xv = row[q];
            acc[4 * q] = fmaf(v, xv.x, acc[4 * q]);
            acc[4 * q + 1] = fmaf(v, xv.y, acc[4 * q + 1]);
            acc[4 * q + 2] = fmaf(v, xv.z, acc[4 * q + 2]);
            acc[4 * q + 3] = fmaf(v, xv.w, acc[4 * q + 3]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < HL_TOKENS; ++tt)
        if (t0 + tt < tokens)
            out[(int64_t)(t0 + tt) * heads * outs + h * outs + o] = from_float<TO>(acc[tt]);
}

// The same for the few tokens of a decode step, where the matrices have to be streamed once
// and few blocks with long chains of loads would do it slowly: a block computes 32 outputs
// of one head for up to 8 tokens, its four warps each taking a quarter of the inputs i; the
// quarters are added in a fixed order through shared memory.
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(128)
head_linear_few_kernel(const TX* __restrict__ x, int ld, int offset, const TW* __restrict__ w,
                       TO* __restrict__ out, int tokens, int heads, int in, int outs) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float fs[];            // x: [in][8], then partial sums
    float* x_s = fs;
    float* part = fs + in * 8;                              // [4][8][32]
    const int per = (outs + 31) / 32;
    const int otile = blockIdx.x % per;
    const int h = blockIdx.x / per;
    const int t0 = blockIdx.y * 8;
    for (int idx = threadIdx.x; idx < 8 * in; idx += blockDim.x) {
        const int tt = idx / in, i = idx - tt * in;
        x_s[i * 8 + tt] =
            t0 + tt < tokens ? to_float(x[(int64_t)(t0 + tt) * ld + offset + h * in + i]) : 0.f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int o = otile * 32 + lane;
    const int quarter = (in + 3) / 4;
    const int i0 = slice * quarter, i1 = min(in, i0 + quarter);
    float acc[8];
#pragma unroll
    for (int tt = 0; tt < 8; ++tt) acc[tt] = 0.f;
    if (o < outs) {
        const TW* wh = w + (int64_t)h * in * outs + o;
#pragma unroll 8
        for (int i = i0; i < i1; ++i) {
            const float v = to_float(wh[(int64_t)i * outs]);
            const float4 x0 = *reinterpret_cast<const float4*>(x_s + i * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(x_s + i * 8 + 4);
            acc[0] = fmaf(v, x0.x, acc[0]); acc[1] = fmaf(v, x0.y, acc[1]);
            acc[2] = fmaf(v, x0.z, acc[2]); acc[3] = fmaf(v, x0.w, acc[3]);
            acc[4] = fmaf(v, x1.x, acc[4]); acc[5] = fmaf(v, x1.y, acc[5]);
            acc[6] = fmaf(v, x1.z, acc[6]); acc[7] = fmaf(v, x1.w, acc[7]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < 8; ++tt) part[(slice * 8 + tt) * 32 + lane] = acc[tt];
    __syncthreads();
    for (int idx = threadIdx.x; idx < 8 * 32; idx += blockDim.x) {
        const int l = idx & 31, tt = idx >> 5;
        const int oo = otile * 32 + l;
        if (oo >= outs || t0 + tt >= tokens) continue;
        float v = 0.f;
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) v += part[(sl * 8 + tt) * 32 + l];
        out[(int64_t)(t0 + tt) * heads * outs + h * outs + oo] = from_float<TO>(v);
    }
}

template <typename TX, typename TW, typename TO>
int launch_head_linear(const void* x, int ld, int offset, const void* w, void* out, int tokens,
                       int heads, int in, int outs, cudaStream_t s) {
    const bool few = tokens <= 16;
    const int tile = few ? 8 : 16;
    const size_t smem = (size_t)tile * in * sizeof(float) + (few ? 4 * 8 * 32 * sizeof(float) : 0);
    if (smem > 48 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    const int rows = (tokens + tile - 1) / tile;
    if (rows > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid(((outs + 127) / 128) * heads, rows);
    if (few) {
        dim3 few_grid(((outs + 31) / 32) * heads, rows);
        MB_LAUNCH((head_linear_few_kernel<TX, TW, TO>), few_grid, 128, smem, s, (const TX*)x, ld, offset,
                  (const TW*)w, (TO*)out, tokens, heads, in, outs);
    } else
        MB_LAUNCH((head_linear_kernel<TX, TW, TO, 16>), grid, 128, smem, s, (const TX*)x, ld, offset,
                  (const TW*)w, (TO*)out, tokens, heads, in, outs);
    return launch_status();
}


// A pair of numbers turned by the angle of (position, pair i): (u, v) -> (u cos - v sin, v cos +
// u sin); cos_t and sin_t are [positions][pairs].
__device__ __forceinline__ void turn_pair(float& u, float& v, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int pos, int pairs, int i) {
    const float c = cos_t[(int64_t)pos * pairs + i], s = sin_t[(int64_t)pos * pairs + i];
    const float a = u * c - v * s, b = v * c + u * s;
    u = a;
    v = b;
}

// What stands in front of latent attention with a query latent and a rotated key part shared
// by the heads. A warp per token, float32 arithmetic:
//   narrow[t] = rmsnorm(pre[t][0 .. q_rank)) * wq                         (if q_rank > 0)
//   page row of t = [rmsnorm(pre[t][kv .. kv + rank)) * wc | rot(pre[t][kv + rank .. + rot_dim))]
//                                                                       (if pages are given)
// The rotation pairs neighbours (2i, 2i + 1) when `interleaved`, else i with i + rot_dim / 2.
template <typename T>
__global__ void latent_prepare_kernel(const float* __restrict__ pre, int ld, int q_rank,
                                      const void* __restrict__ wq, T* __restrict__ narrow,
                                      int kv, int rank, const void* __restrict__ wc, int w_dtype,
                                      int rot_dim, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int interleaved, float eps,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token,
                                      const int* __restrict__ table, int max_pages,
                                      T* __restrict__ pages, int page_size, int tokens) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const int seq = seq_of_token[t];
    const float* row = pre + (int64_t)t * ld;
    if (q_rank > 0) {
        float ss = 0.f;
        if (seq >= 0)
            for (int c = lane; c < q_rank; c += 32) ss = fmaf(row[c], row[c], ss);
        ss = warp_sum(ss);
        const float rstd = 1.f / sqrtf(ss / (float)q_rank + eps);
        for (int c = lane; c < q_rank; c += 32)
            narrow[(int64_t)t * q_rank + c] =
                from_float<T>(seq >= 0 ? row[c] * rstd * load_as_float(wq, c, w_dtype) : 0.f);
    }
    if (pages == nullptr || seq < 0) return;
    const int pos = positions[t];
    const int page = table_page(table, seq, max_pages, pos / page_size);
    if (page < 0) return;
    const float* x = row + kv;
    float ss = 0.f;
    for (int c = lane; c < rank; c += 32) ss = fmaf(x[c], x[c], ss);
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)rank + eps);
    T* to = pages + ((int64_t)page * page_size + (pos % page_size)) * (rank + rot_dim);
    for (int c = lane; c < rank; c += 32)
        to[c] = from_float<T>(x[c] * rstd * load_as_float(wc, c, w_dtype));
    const int pairs = rot_dim / 2, at = checked_position(pos);
    for (int i = lane; i < pairs; i += 32) {
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + pairs;
        float u = x[rank + a], v = x[rank + b];
        turn_pair(u, v, cos_t, sin_t, at, pairs, i);
        to[rank + a] = from_float<T>(u);
        to[rank + b] = from_float<T>(v);
    }
}

// In place: the rot_dim numbers from column `offset` of every head's row of q [tokens][heads *
// row] turned by the token's position. A thread per (token, head, pair).
template <typename T>
__global__ void rope_rows_kernel(T* __restrict__ q, int heads, int row, int offset, int rot_dim,
                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 int interleaved, const int* __restrict__ positions,
                                 const int* __restrict__ seq_of_token, int tokens) {
    grid_dependency_sync();
    const int pairs = rot_dim / 2;
    const int64_t id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (int64_t)tokens * heads * pairs) return;
    const int i = (int)(id % pairs);
    const int h = (int)((id / pairs) % heads);
    const int t = (int)(id / ((int64_t)pairs * heads));
    if (seq_of_token[t] < 0) return;
    const int pos = checked_position(positions[t]);
    T* at = q + ((int64_t)t * heads + h) * row + offset;
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + pairs;
    float u = to_float(at[a]), v = to_float(at[b]);
    turn_pair(u, v, cos_t, sin_t, pos, pairs, i);
    at[a] = from_float<T>(u);
    at[b] = from_float<T>(v);
}

}  // namespace mb

using namespace mb;

// dtype: the pages' type (MB_F32 or MB_BF16); w_dtype: the norm weight's.
MB_EXPORT int mb_latent_norm_store(const float* pre, int ld, int offset, const void* w, int w_dtype,
                                   float eps, const int* positions, const int* seq_of_token,
                                   const int* table, int max_pages, void* pages, int rank,
                                   int page_size, int tokens, int dtype, void* stream) {
    if (tokens <= 0 || rank <= 0) return MB_OK;
    if (page_size <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    const int blocks = (tokens + 3) / 4;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((latent_norm_store_kernel<float>), blocks, 128, 0, s, pre, ld, offset, w, w_dtype, eps,
                  positions, seq_of_token, table, max_pages, (float*)pages, rank, page_size, tokens);
    else if (dtype == MB_BF16)
        MB_LAUNCH((latent_norm_store_kernel<__nv_bfloat16>), blocks, 128, 0, s, pre, ld, offset, w,
                  w_dtype, eps, positions, seq_of_token, table, max_pages, (__nv_bfloat16*)pages, rank,
                  page_size, tokens);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

// x [tokens][ld] (its heads from column `offset`), w [heads][in][outs], out [tokens][heads *
// outs]; each of the three float32 or bfloat16.
MB_EXPORT int mb_head_linear(const void* x, int x_dtype, int ld, int offset, const void* w,
                             int w_dtype, void* out, int out_dtype, int tokens, int heads, int in,
                             int outs, void* stream) {
    if (tokens <= 0 || heads <= 0) return MB_OK;
    if (in <= 0 || outs <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case 0: return launch_head_linear<float, float, float>(x, ld, offset, w, out, tokens, heads, in, outs, s);
        case 3: return launch_head_linear<float, bf, bf>(x, ld, offset, w, out, tokens, heads, in, outs, s);
        case 7: return launch_head_linear<bf, bf, bf>(x, ld, offset, w, out, tokens, heads, in, outs, s);
        case 2: return launch_head_linear<float, bf, float>(x, ld, offset, w, out, tokens, heads, in, outs, s);
        case 1: return launch_head_linear<float, float, bf>(x, ld, offset, w, out, tokens, heads, in, outs, s);
    }
    return MB_ERR_BAD_DTYPE;
}

// dtype: the type of `narrow` and of the pages (MB_F32 or MB_BF16); w_dtype: the type of both
// norm weights. q_rank 0: no query latent; pages null: the layer stores no rows; rot_dim 0: no
// rotated part (cos_t and sin_t may then be null).
MB_EXPORT int mb_latent_prepare(const float* pre, int ld, int q_rank, const void* wq, void* narrow,
                                int kv, int rank, const void* wc, int w_dtype, int rot_dim,
                                const float* cos_t, const float* sin_t, int interleaved, float eps,
                                const int* positions, const int* seq_of_token, const int* table,
                                int max_pages, void* pages, int page_size, int tokens, int dtype,
                                void* stream) {
    if (tokens <= 0) return MB_OK;
    if (q_rank < 0 || rot_dim < 0 || (rot_dim & 1)) return MB_ERR_UNSUPPORTED_SIZE;
    if (pages != nullptr && (rank <= 0 || page_size <= 0 || (rot_dim > 0 && (!cos_t || !sin_t))))
        return MB_ERR_UNSUPPORTED_SIZE;
    const int blocks = (tokens + 3) / 4;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((latent_prepare_kernel<float>), blocks, 128, 0, s, pre, ld, q_rank, wq, (float*)narrow,
                  kv, rank, wc, w_dtype, rot_dim, cos_t, sin_t, interleaved, eps, positions,
                  seq_of_token, table, max_pages, (float*)pages, page_size, tokens);
    else if (dtype == MB_BF16)
        MB_LAUNCH((latent_prepare_kernel<__nv_bfloat16>), blocks, 128, 0, s, pre, ld, q_rank, wq,
                  (__nv_bfloat16*)narrow, kv, rank, wc, w_dtype, rot_dim, cos_t, sin_t, interleaved, eps,
                  positions, seq_of_token, table, max_pages, (__nv_bfloat16*)pages, page_size, tokens);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

MB_EXPORT int mb_rope_rows(void* q, int dtype, int heads, int row, int offset, int rot_dim,
                           const float* cos_t, const float* sin_t, int interleaved,
                           const int* positions, const int* seq_of_token, int tokens, void* stream) {
    if (tokens <= 0 || rot_dim <= 0) return MB_OK;
    if ((rot_dim & 1) || offset < 0 || offset + rot_dim > row || heads <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    const long long total = (long long)tokens * heads * (rot_dim / 2);
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((rope_rows_kernel<float>), (int)blocks, 256, 0, s, (float*)q, heads, row, offset,
                  rot_dim, cos_t, sin_t, interleaved, positions, seq_of_token, tokens);
    else if (dtype == MB_BF16)
        MB_LAUNCH((rope_rows_kernel<__nv_bfloat16>), (int)blocks, 256, 0, s, (__nv_bfloat16*)q, heads,
                  row, offset, rot_dim, cos_t, sin_t, interleaved, positions, seq_of_token, tokens);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}
