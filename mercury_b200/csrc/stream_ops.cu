// Operations on the float32 residual stream and the logits: an embedding lookup with a
// constant factor, the residual sum under a per-feature scale fused with the norm that follows
// (layer norm or RMS norm), the soft cap of the logits, the norm behind two sublayers that ran
// side by side, and the short causal convolution of the stream that a sublayer may read in
// place of the stream. All arithmetic is float32.
#include "common.cuh"

namespace mb {

// out[t, :] = table[ids[t], :] * scale, written into the float32 residual stream.
__global__ void embed_scaled_kernel(const int* __restrict__ ids, const void* __restrict__ table,
                                    int table_dtype, float scale, float* __restrict__ out,
                                    int hidden, int vocab) {
    grid_dependency_sync();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
#ifdef MB_BOUNDS_CHECK
    if (!ok && threadIdx.x == 0) check_report(MB_CHECK_TOKEN, id, vocab);
#endif
    const int64_t base = (int64_t)(ok ? id : 0) * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[(int64_t)t * hidden + c] = ok ? load_as_float(table, base + c, table_dtype) * scale : 0.f;
}

// h <- h + delta * scale (delta and scale optional; scale one number per feature), then, when
// a norm weight is given, out = (x - mean) / sqrt(var + eps) * w of the new row (center = 1;
// var is the mean of the squared deviations) or x / sqrt(mean(x^2) + eps) * w (center = 0).
// With `rows` only the rows listed are normalised (out row r from stream row rows[r]) and
// the stream is left as it was. One block per row; the row stays in shared memory between
// the sums, so mean and variance are taken in two passes over the same numbers.
template <typename TD, typename TO>
__global__ void scaled_add_norm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const void* __restrict__ scale, int scale_dtype,
                                       const void* __restrict__ w, int w_dtype, float eps,
                                       int center, TO* __restrict__ out,
                                       const int* __restrict__ rows, int hidden) {
    grid_dependency_sync();
    extern __shared__ float row_s[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = (int64_t)(rows ? rows[r] : r) * hidden;
    const int64_t dst = (int64_t)r * hidden;
    float sum = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float x = h[src + c];
        if (delta) {
            const float s = scale ? load_as_float(scale, c, scale_dtype) : 1.f;
            x = fmaf(to_float(delta[src + c]), s, x);
            if (!rows) h[src + c] = x;
        }
        row_s[c] = x;
        sum += x;
    }
    if (w == nullptr) return;
    float mean = 0.f;
    if (center) mean = block_sum(sum, scratch) / (float)hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float d = row_s[c] - mean;
        ss += d * d;
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(ss / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[dst + c] = from_float<TO>((row_s[c] - mean) * rstd * load_as_float(w, c, w_dtype));
}

// x <- cap * tanh(x / cap)
__global__ void softcap_kernel(float* __restrict__ x, int64_t total, float cap) {
    grid_dependency_sync();
    const float inv = 1.f / cap;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}


// A norm BEHIND two sublayers that ran side by side: d = a * delta + b * delta2 (delta2 may be
// null), h <- h + d * rsqrt(mean(d^2) + eps) * w. One block per row, d kept in shared memory.
// With a ring (the state of the convolution in front of the sublayer, [slots][span][hidden]),
// the row of the stream as the sublayer found it is first kept there if it is among its
// sequence's last `span` positions (at position modulo span): the kernel that read the ring
// ran earlier on the stream, and this one sees the old row anyway.
template <typename TD>
__global__ void rmsnorm_add_pair_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                        const TD* __restrict__ delta2, float a, float b,
                                        const void* __restrict__ w, int w_dtype, float eps,
                                        int hidden, float* __restrict__ ring, int64_t ring_stride,
                                        int span, const int* __restrict__ positions,
                                        const int* __restrict__ seq_of_token,
                                        const int* __restrict__ kv_len, const int* __restrict__ slots) {
    grid_dependency_sync();
    extern __shared__ float pair_row_s[];
    __shared__ float scratch[33];
    const int64_t at = (int64_t)blockIdx.x * hidden;
    float* keep = nullptr;
    if (ring != nullptr) {
        const int seq = seq_of_token[blockIdx.x];
        if (seq >= 0) {
            const int pos = positions[blockIdx.x];
            if (pos >= kv_len[seq] - span)
                keep = ring + (int64_t)slots[seq] * ring_stride + (int64_t)(pos % span) * hidden;
        }
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float d = a * to_float(delta[at + c]);
        if (delta2 != nullptr) d = fmaf(b, to_float(delta2[at + c]), d);
        pair_row_s[c] = d;
        ss = fmaf(d, d, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(ss / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float old = h[at + c];
        if (keep != nullptr) keep[c] = old;
        h[at + c] = old + pair_row_s[c] * rstd * load_as_float(w, c, w_dtype);
    }
}

// Two sublayer outputs that ran side by side, each under an RMS norm of its own, joined and
// sent through the norm behind the sublayer: with n(x) = x * rsqrt(mean(x^2) + eps) * wx (or x
// itself where wx is null), z = a n(x) + b n(y), h <- h + z * rsqrt(mean(z^2) + eps) * w, and,
// when the norm that follows is given, out = h * rsqrt(mean(h^2) + eps2) * w2 of the new h in
// the same pass. One block per row, the rows kept in shared memory between the sums. All
// weights float32.
template <typename TD, typename TO>
__global__ void rmsnorm_join_add_kernel(float* __restrict__ h, const TD* __restrict__ x,
                                        const TD* __restrict__ y, const float* __restrict__ wx,
                                        const float* __restrict__ wy, float a, float b,
                                        const float* __restrict__ w, float eps,
                                        const float* __restrict__ w2, float eps2,
                                        TO* __restrict__ out, int hidden) {
    grid_dependency_sync();
    extern __shared__ float join_s[];
    float* x_s = join_s;
    float* y_s = join_s + hidden;
    __shared__ float scratch[33];
    const int64_t at = (int64_t)blockIdx.x * hidden;
    float sx = 0.f, sy = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float xv = to_float(x[at + c]), yv = to_float(y[at + c]);
        x_s[c] = xv;
        y_s[c] = yv;
        sx = fmaf(xv, xv, sx);
        sy = fmaf(yv, yv, sy);
    }
    float rx = 1.f, ry = 1.f;
    if (wx != nullptr) rx = 1.f / sqrtf(block_sum(sx, scratch) / (float)hidden + eps);
    if (wy != nullptr) ry = 1.f / sqrtf(block_sum(sy, scratch) / (float)hidden + eps);
    float sz = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float xn = wx != nullptr ? x_s[c] * rx * wx[c] : x_s[c];
        const float yn = wy != nullptr ? y_s[c] * ry * wy[c] : y_s[c];
        const float z = fmaf(b, yn, a * xn);
        x_s[c] = z;
        sz = fmaf(z, z, sz);
    }
    const float rz = 1.f / sqrtf(block_sum(sz, scratch) / (float)hidden + eps);
    float sh = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = h[at + c] + x_s[c] * rz * w[c];
        h[at + c] = v;
        y_s[c] = v;
        sh = fmaf(v, v, sh);
    }
    if (w2 == nullptr) return;
    const float rh = 1.f / sqrtf(block_sum(sh, scratch) / (float)hidden + eps2);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[at + c] = from_float<TO>(y_s[c] * rh * w2[c]);
}

// What a sublayer reads in place of the stream: out[t][c] = x[t][c] + sum_j w[c][j] *
// x(p - taps + 1 + j)[c], where x(q) is the stream's row at position q of the token's
// sequence: zero for q < 0, a row of this step for q >= first (the position of the
// sequence's first token in this step), else ring[slot][q % (taps - 1)], the rows that
// earlier steps left. The ring is not changed here. w null: out = x. A thread per (token,
// channel); float32 arithmetic, j ascending, so a token's sum does not depend on the cut.
template <typename TO>
__global__ void stream_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, int taps,
                                   const float* __restrict__ ring, int64_t ring_stride,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ seq_of_token,
                                   const int* __restrict__ q_start, const int* __restrict__ kv_len,
                                   const int* __restrict__ slots, TO* __restrict__ out, int tokens,
                                   int hidden) {
    grid_dependency_sync();
    const int t = blockIdx.y;
    const int seq = seq_of_token[t];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= hidden) return;
    if (seq < 0) {
        out[(int64_t)t * hidden + c] = from_float<TO>(0.f);
        return;
    }
    const float own = x[(int64_t)t * hidden + c];
    if (w == nullptr) {
        out[(int64_t)t * hidden + c] = from_float<TO>(own);
        return;
    }
    const int pos = positions[t];
    const int first = kv_len[seq] - (q_start[seq + 1] - q_start[seq]);
    const int span = taps - 1;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = span - j;                 // how many tokens before this one
        const int q = pos - back;
        float v = 0.f;
        if (back == 0) v = own;
        else if (q >= first) v = x[(int64_t)(t - back) * hidden + c];
        else if (q >= 0) v = ring[(int64_t)slots[seq] * ring_stride + (int64_t)(q % span) * hidden + c];
        acc = fmaf(w[(int64_t)c * taps + j], v, acc);
    }
    out[(int64_t)t * hidden + c] = from_float<TO>(own + acc);
}

// After the step's convolutions: the stream's rows at each sequence's last taps - 1
// positions of this step into its ring, row of position q at q % (taps - 1).
__global__ void stream_tail_store_kernel(const float* __restrict__ x, float* __restrict__ ring,
                                         int64_t ring_stride, int span,
                                         const int* __restrict__ q_start,
                                         const int* __restrict__ kv_len,
                                         const int* __restrict__ slots, int hidden) {
    grid_dependency_sync();
    const int seq = blockIdx.y;
    const int begin = q_start[seq], end = q_start[seq + 1];
    const int back = blockIdx.z + 1;               // the back-th token from the step's end
    if (end - begin < back) return;
    const int t = end - back;
    const int pos = kv_len[seq] - back;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= hidden) return;
    ring[(int64_t)slots[seq] * ring_stride + (int64_t)(pos % span) * hidden + c] =
        x[(int64_t)t * hidden + c];
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_embed_scaled(const int* ids, const void* table, int table_dtype, float scale,
                              float* out, int tokens, int hidden, int vocab, void* stream) {
    if (tokens <= 0) return MB_OK;
    MB_LAUNCH((embed_scaled_kernel), tokens, 256, 0, (cudaStream_t)stream, ids, table, table_dtype,
              scale, out, hidden, vocab);
    return launch_status();
}

// delta_dtype / out_dtype: MB_F32 or MB_BF16. delta, scale, w, out and rows may each be null
// (w null: only the sum is made; out is then not touched).
MB_EXPORT int mb_scaled_add_norm(float* h, const void* delta, int delta_dtype, const void* scale,
                                 int scale_dtype, const void* w, int w_dtype, float eps, int center,
                                 void* out, int out_dtype, const int* rows, int count, int hidden,
                                 void* stream) {
    if (count <= 0 || hidden <= 0) return MB_OK;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 160 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define MB_SAN_CASE(TD, TO)                                                                       \
    do {                                                                                          \
        static size_t raised = 0;                                                                 \
        if (smem + 256 > 48 * 1024 && smem > raised) {                                                \
            if (cudaFuncSetAttribute(scaled_add_norm_kernel<TD, TO>,                              \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=   \
                cudaSuccess)                                                                      \
                return MB_ERR_UNSUPPORTED_SIZE;                                                   \
            raised = smem;                                                                        \
        }                                                                                         \
        MB_LAUNCH((scaled_add_norm_kernel<TD, TO>), count, threads, smem, s, h, (const TD*)delta, \
                  scale, scale_dtype, w, w_dtype, eps, center, (TO*)out, rows, hidden);           \
    } while (0)
    if (delta_dtype == MB_F32 && out_dtype == MB_F32) MB_SAN_CASE(float, float);
    else if (delta_dtype == MB_F32 && out_dtype == MB_BF16) MB_SAN_CASE(float, bf);
    else if (delta_dtype == MB_BF16 && out_dtype == MB_F32) MB_SAN_CASE(bf, float);
    else if (delta_dtype == MB_BF16 && out_dtype == MB_BF16) MB_SAN_CASE(bf, bf);
    else return MB_ERR_BAD_DTYPE;
#undef MB_SAN_CASE
    return launch_status();
}

MB_EXPORT int mb_softcap(float* x, long long total, float cap, void* stream) {
    if (total <= 0) return MB_OK;
    if (!(cap > 0.f)) return MB_ERR_UNSUPPORTED_SIZE;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    MB_LAUNCH((softcap_kernel), blocks, 256, 0, (cudaStream_t)stream, x, (int64_t)total, cap);
    return launch_status();
}

// delta2 may be null (then b is not used); both deltas share `delta_dtype`.
MB_EXPORT int mb_rmsnorm_add_pair(float* h, const void* delta, const void* delta2, int delta_dtype,
                                  float a, float b, const void* w, int w_dtype, float eps, int count,
                                  int hidden, float* ring, long long ring_stride, int span,
                                  const int* positions, const int* seq_of_token, const int* kv_len,
                                  const int* slots, void* stream) {
    if (count <= 0 || hidden <= 0) return MB_OK;
    if (ring != nullptr && (span <= 0 || !positions || !seq_of_token || !kv_len || !slots))
        return MB_ERR_UNSUPPORTED_SIZE;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 160 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define MB_RAP_CASE(TD)                                                                           \
    do {                                                                                          \
        static size_t raised = 0;                                                                 \
        if (smem + 256 > 48 * 1024 && smem > raised) {                                                \
            if (cudaFuncSetAttribute(rmsnorm_add_pair_kernel<TD>,                                 \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=   \
                cudaSuccess)                                                                      \
                return MB_ERR_UNSUPPORTED_SIZE;                                                   \
            raised = smem;                                                                        \
        }                                                                                         \
        MB_LAUNCH((rmsnorm_add_pair_kernel<TD>), count, threads, smem, s, h, (const TD*)delta,    \
                  (const TD*)delta2, a, b, w, w_dtype, eps, hidden, ring, (int64_t)ring_stride,   \
                  span, positions, seq_of_token, kv_len, slots);                                  \
    } while (0)
    if (delta_dtype == MB_F32) MB_RAP_CASE(float);
    else if (delta_dtype == MB_BF16) MB_RAP_CASE(bf);
    else return MB_ERR_BAD_DTYPE;
#undef MB_RAP_CASE
    return launch_status();
}

// x, y: [count][hidden] of x_dtype; wx, wy (null: that side is not normed), w and w2 (null: no
// norm computed ahead) float32 [hidden]; out of out_dtype.
MB_EXPORT int mb_rmsnorm_join_add(float* h, const void* x, const void* y, int x_dtype, const float* wx,
                                  const float* wy, float a, float b, const float* w, float eps,
                                  const float* w2, float eps2, void* out, int out_dtype, int count,
                                  int hidden, void* stream) {
    if (count <= 0 || hidden <= 0) return MB_OK;
    if (!x || !y || !w || (w2 != nullptr && !out)) return MB_ERR_UNSUPPORTED_SIZE;
    const size_t smem = (size_t)2 * hidden * sizeof(float);
    if (smem > 160 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define MB_RJ_CASE(TD, TO)                                                                        \
    do {                                                                                          \
        static size_t raised = 0;                                                                 \
        if (smem + 256 > 48 * 1024 && smem > raised) {                                            \
            if (cudaFuncSetAttribute(rmsnorm_join_add_kernel<TD, TO>,                             \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=   \
                cudaSuccess)                                                                      \
                return MB_ERR_UNSUPPORTED_SIZE;                                                   \
            raised = smem;                                                                        \
        }                                                                                         \
        MB_LAUNCH((rmsnorm_join_add_kernel<TD, TO>), count, threads, smem, s, h, (const TD*)x,    \
                  (const TD*)y, wx, wy, a, b, w, eps, w2, eps2, (TO*)out, hidden);                \
    } while (0)
    const bool wide_out = w2 == nullptr || out_dtype == MB_F32;
    if (w2 != nullptr && out_dtype != MB_F32 && out_dtype != MB_BF16) return MB_ERR_BAD_DTYPE;
    if (x_dtype == MB_F32 && wide_out) MB_RJ_CASE(float, float);
    else if (x_dtype == MB_F32) MB_RJ_CASE(float, bf);
    else if (x_dtype == MB_BF16 && wide_out) MB_RJ_CASE(bf, float);
    else if (x_dtype == MB_BF16) MB_RJ_CASE(bf, bf);
    else return MB_ERR_BAD_DTYPE;
#undef MB_RJ_CASE
    return launch_status();
}

// w: [hidden][taps] float32 or null (out = x); ring: [slots][taps - 1][hidden] float32 with
// `ring_stride` floats between two slots (null when taps is 1). out_dtype: MB_F32 or MB_BF16.
MB_EXPORT int mb_stream_conv(const float* x, const float* w, int taps, const float* ring,
                             long long ring_stride, const int* positions, const int* seq_of_token,
                             const int* q_start, const int* kv_len, const int* slots, void* out,
                             int out_dtype, int tokens, int hidden, void* stream) {
    if (tokens <= 0 || hidden <= 0) return MB_OK;
    if (w != nullptr && (taps < 1 || (taps > 1 && ring == nullptr))) return MB_ERR_UNSUPPORTED_SIZE;
    if (tokens > 65535 * 16) return MB_ERR_UNSUPPORTED_SIZE;
    const int threads = hidden >= 256 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    for (int t0 = 0; t0 < tokens; t0 += 65535) {
        const int n = tokens - t0 < 65535 ? tokens - t0 : 65535;
        dim3 grid((hidden + threads - 1) / threads, n);
        const float* xs = x + (int64_t)t0 * hidden;
        if (out_dtype == MB_F32)
            MB_LAUNCH((stream_conv_kernel<float>), grid, threads, 0, s, xs, w, taps, ring,
                      (int64_t)ring_stride, positions + t0, seq_of_token + t0, q_start, kv_len, slots,
                      (float*)out + (int64_t)t0 * hidden, n, hidden);
        else if (out_dtype == MB_BF16)
            MB_LAUNCH((stream_conv_kernel<__nv_bfloat16>), grid, threads, 0, s, xs, w, taps, ring,
                      (int64_t)ring_stride, positions + t0, seq_of_token + t0, q_start, kv_len, slots,
                      (__nv_bfloat16*)out + (int64_t)t0 * hidden, n, hidden);
        else
            return MB_ERR_BAD_DTYPE;
    }
    return launch_status();
}

MB_EXPORT int mb_stream_tail_store(const float* x, float* ring, long long ring_stride, int span,
                                   const int* q_start, const int* kv_len, const int* slots,
                                   int num_seqs, int hidden, void* stream) {
    if (num_seqs <= 0 || hidden <= 0 || span <= 0) return MB_OK;
    if (num_seqs > 65535 || span > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    const int threads = hidden >= 256 ? 256 : 128;
    dim3 grid((hidden + threads - 1) / threads, num_seqs, span);
    MB_LAUNCH((stream_tail_store_kernel), grid, threads, 0, (cudaStream_t)stream, x, ring,
              (int64_t)ring_stride, span, q_start, kv_len, slots, hidden);
    return launch_status();
}
