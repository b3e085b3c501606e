// Grouped-query attention whose weights are sigmoids, not a softmax: the weight of a seen key
// is sigmoid(q . k * scale + b_h), b_h one number per query head, and the weights are not
// normalised over the keys, so a row's output is a plain sum over its keys and key ranges
// add up without a merge. Key j is seen from position p iff j <= p and (p - j < window or j <
// keep_first): a sliding window beside first tokens that stay visible (window 0: every key).
//
// In front of it: per-head RMS norms of queries and keys (one weight of `d` numbers shared by
// the heads), the rotation of the first rot_dim numbers of each head, and the store of keys
// and values into the pages; the values may be the keys as projected (before norm and
// rotation).
//
// Work split as in attention_simt.cu: the (query token, head of the group) pairs of one
// sequence and one KV head are rows, a block of 8 warps takes 16 of them, keys are walked in
// tiles of 32 aligned to absolute positions, one key per lane for the scores and 32 features
// per lane for the weighted sum. A block walks the tiles of the kept first tokens and then
// those of its rows' windows (no tile twice). With num_splits > 1 the tiles are dealt over
// gridDim.z and the partial sums are added in a fixed order by a second kernel. Scores,
// sigmoids and sums are float32.
#include "common.cuh"
#include "mma_sync.cuh"

namespace mb {

constexpr int SG_ROWS = 16;
constexpr int SG_WARPS = 8;
constexpr int SG_RPW = SG_ROWS / SG_WARPS;
constexpr int SG_KEYS = 32;

// pre: [tokens][ld] float32 = [q (n_q * d) | k (n_kv * d) | v (n_kv * dv), unless the values are
// the keys]. A warp per (token, head), heads counted over q heads, then k heads, then v heads.
template <typename T>
__global__ void qk_norm_rope_store_kernel(const float* __restrict__ pre, int ld,
                                          const float* __restrict__ wq, const float* __restrict__ wk,
                                          float eps, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int rot_dim,
                                          int interleaved, const int* __restrict__ positions,
                                          const int* __restrict__ seq_of_token,
                                          const int* __restrict__ table, int max_pages,
                                          T* __restrict__ k_pages, T* __restrict__ v_pages,
                                          T* __restrict__ q_out, int n_q, int n_kv, int d, int dv,
                                          int values_are_keys, int page_size, int tokens) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const int per_token = n_q + n_kv + (values_are_keys ? 0 : n_kv);
    const int64_t id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (id >= (int64_t)tokens * per_token) return;
    const int t = (int)(id / per_token), slot = (int)(id - (int64_t)t * per_token);
    const int seq = seq_of_token[t];
    if (seq < 0) {
        if (slot < n_q)
            for (int c = lane; c < d; c += 32) q_out[((int64_t)t * n_q + slot) * d + c] = from_float<T>(0.f);
        return;
    }
    const int pos = positions[t];
    const float* row = pre + (int64_t)t * ld;
    if (slot >= n_q + n_kv) {                     // a value head of its own: stored as projected
        const int h = slot - n_q - n_kv;
        const int page = table_page(table, seq, max_pages, pos / page_size);
        if (page < 0) return;
        const float* x = row + (n_q + n_kv) * d + h * dv;
        T* to = v_pages + (((int64_t)page * n_kv + h) * page_size + (pos % page_size)) * dv;
        for (int c = lane; c < dv; c += 32) to[c] = from_float<T>(x[c]);
        return;
    }
    const bool is_q = slot < n_q;
    const int h = is_q ? slot : slot - n_q;
    const float* x = row + (is_q ? 0 : n_q * d) + h * d;
    T* to;
    if (is_q) {
        to = q_out + ((int64_t)t * n_q + h) * d;
    } else {
        const int page = table_page(table, seq, max_pages, pos / page_size);
        if (page < 0) return;
        const int64_t at = ((int64_t)page * n_kv + h) * page_size + (pos % page_size);
        to = k_pages + at * d;
        if (values_are_keys) {
            T* vto = v_pages + at * d;
            for (int c = lane; c < d; c += 32) vto[c] = from_float<T>(x[c]);
        }
    }
    const float* w = is_q ? wq : wk;
    float rstd = 1.f;
    if (w != nullptr) {
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) ss = fmaf(x[c], x[c], ss);
        ss = warp_sum(ss);
        rstd = 1.f / sqrtf(ss / (float)d + eps);
    }
    const int pairs = rot_dim / 2, at_pos = checked_position(pos);
    for (int i = lane; i < pairs; i += 32) {
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + pairs;
        float u = x[a] * rstd, v = x[b] * rstd;
        if (w != nullptr) {
            u *= w[a];
            v *= w[b];
        }
        const float c = cos_t[(int64_t)at_pos * pairs + i], s = sin_t[(int64_t)at_pos * pairs + i];
        to[a] = from_float<T>(u * c - v * s);
        to[b] = from_float<T>(v * c + u * s);
    }
    for (int c = rot_dim + lane; c < d; c += 32)
        to[c] = from_float<T>(w != nullptr ? x[c] * rstd * w[c] : x[c]);
}

template <typename T, int NC>
__global__ void __launch_bounds__(SG_WARPS * 32)
sigmoid_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ table, int max_pages,
                         const int* __restrict__ q_start, const int* __restrict__ kv_len_of,
                         const float* __restrict__ head_bias, T* __restrict__ out,
                         float* __restrict__ part, int n_q, int n_kv, int d, int page_size,
                         float scale, int window, int keep_first, int tiles_per_seq, int num_splits) {
    grid_dependency_sync();
    extern __shared__ float smem[];
    const int seq = blockIdx.x / tiles_per_seq;
    const int tile = blockIdx.x - seq * tiles_per_seq;
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    const int group = n_q / n_kv;
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    const int row0 = tile * SG_ROWS;
    if (row0 >= q_len * group) return;
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;

    float* q_s = smem;                                   // [SG_ROWS][d]
    float* k_s = q_s + SG_ROWS * d;                      // [SG_KEYS][d + 1]
    float* v_s = k_s + SG_KEYS * (d + 1);                // [SG_KEYS][d]
    int* page_s = reinterpret_cast<int*>(v_s + SG_KEYS * d);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int idx = tid; idx < SG_ROWS * d; idx += blockDim.x) {
        const int r = idx / d, c = idx - r * d;
        const int row = row0 + r;
        const int tok = row / group, hg = row - tok * group;
        q_s[idx] = tok < q_len ? to_float(q[((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * d + c]) : 0.f;
    }
    int row_pos[SG_RPW];
    bool row_ok[SG_RPW];
    float bias[SG_RPW];
#pragma unroll
    for (int rr = 0; rr < SG_RPW; ++rr) {
        const int row = row0 + warp * SG_RPW + rr;
        const int tok = row / group, hg = row - tok * group;
        row_ok[rr] = tok < q_len;
        row_pos[rr] = first_pos + tok;
        bias[rr] = head_bias[kvh * group + hg];
    }
    // the key tiles of this block: [0, head_hi) for the kept first tokens, [t_lo, t_hi) for the
    // windows; walked as one list with the overlap dropped
    const int tok_min = row0 / group;
    int tok_max = (row0 + SG_ROWS - 1) / group;
    if (tok_max > q_len - 1) tok_max = q_len - 1;
    const int p_min = first_pos + tok_min, p_max = first_pos + tok_max;
    const int t_hi = p_max / SG_KEYS + 1;
    int t_lo = 0;
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / SG_KEYS;
    int head_hi = 0;
    if (window > 0 && keep_first > 0) head_hi = (keep_first + SG_KEYS - 1) / SG_KEYS;
    if (head_hi > t_lo) head_hi = t_lo;                 // the window's tiles take over from t_lo
    const int count = head_hi + (t_hi - t_lo);
    int n_lo = 0, n_hi = count;
    if (num_splits > 1) {
        const int per = (count + num_splits - 1) / num_splits;
        n_lo = split * per;
        n_hi = n_lo + per < count ? n_lo + per : count;
    }

    float acc[SG_RPW][NC];
#pragma unroll
    for (int rr = 0; rr < SG_RPW; ++rr)
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[rr][c] = 0.f;

    for (int n = n_lo; n < n_hi; ++n) {
        const int kt = n < head_hi ? n : t_lo + (n - head_hi);
        __syncthreads();
        if (tid < SG_KEYS) {
            const int key = kt * SG_KEYS + tid;
            int page = -1;
            if (key < kv_len) page = table_page(table, seq, max_pages, key / page_size);
            page_s[tid] = page;
        }
        __syncthreads();
        for (int idx = tid; idx < SG_KEYS * d; idx += blockDim.x) {
            const int j = idx / d, c = idx - j * d;
            const int page = page_s[j];
            float kv = 0.f, vv = 0.f;
            if (page >= 0) {
                const int key = kt * SG_KEYS + j;
                const int64_t at = (((int64_t)page * n_kv + kvh) * page_size + (key % page_size)) * d + c;
                kv = to_float(k_pages[at]);
                vv = to_float(v_pages[at]);
            }
            k_s[j * (d + 1) + c] = kv;
            v_s[idx] = vv;
        }
        __syncthreads();
        float s[SG_RPW];
#pragma unroll
        for (int rr = 0; rr < SG_RPW; ++rr) s[rr] = 0.f;
        const float* krow = k_s + lane * (d + 1);
        const float* qrow = q_s + warp * SG_RPW * d;
        for (int c = 0; c < d; ++c) {
            const float kv = krow[c];
#pragma unroll
            for (int rr = 0; rr < SG_RPW; ++rr) s[rr] = fmaf(qrow[rr * d + c], kv, s[rr]);
        }
        const int key = kt * SG_KEYS + lane;
        const bool key_ok = page_s[lane] >= 0;
#pragma unroll
        for (int rr = 0; rr < SG_RPW; ++rr) {
            bool seen = row_ok[rr] && key_ok && key <= row_pos[rr];
            if (window > 0) seen = seen && (key > row_pos[rr] - window || key < keep_first);
            const float p = seen ? 1.f / (1.f + expf(-(s[rr] * scale + bias[rr]))) : 0.f;
            if (__ballot_sync(0xffffffffu, seen) == 0u) continue;
            for (int j = 0; j < SG_KEYS; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int dim = lane + 32 * c;
                    if (dim < d) acc[rr][c] = fmaf(pj, v_s[j * d + dim], acc[rr][c]);
                }
            }
        }
    }
#pragma unroll
    for (int rr = 0; rr < SG_RPW; ++rr) {
        if (!row_ok[rr]) continue;
        const int row = row0 + warp * SG_RPW + rr;
        const int tok = row / group, hg = row - tok * group;
        const int64_t flat = (int64_t)(q_begin + tok) * n_q + kvh * group + hg;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int dim = lane + 32 * c;
            if (dim >= d) continue;
            if (num_splits == 1) out[flat * d + dim] = from_float<T>(acc[rr][c]);
            else part[(flat * num_splits + split) * d + dim] = acc[rr][c];
        }
    }
}

// out = the sum of a (token, head)'s partial sums, split 0 first.
template <typename T>
__global__ void sigmoid_attention_sum_kernel(const float* __restrict__ part,
                                             const int* __restrict__ seq_of_token,
                                             T* __restrict__ out, int n_q, int d, int num_splits) {
    grid_dependency_sync();
    const int tok = blockIdx.x, head = blockIdx.y;
    const int64_t flat = (int64_t)tok * n_q + head;
    const bool live = seq_of_token[tok] >= 0;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = 0.f;
        if (live)
            for (int z = 0; z < num_splits; ++z) v += part[(flat * num_splits + z) * d + c];
        out[flat * d + c] = from_float<T>(v);
    }
}

template <typename T, int NC>
int launch_sigmoid(const void* q, const void* k_pages, const void* v_pages, const int* table,
                   int max_pages, const int* q_start, const int* kv_len, const float* head_bias,
                   void* out, float* part, int n_q, int n_kv, int d, int page_size, float scale,
                   int window, int keep_first, int num_seqs, int tiles_per_seq, int num_splits,
                   cudaStream_t s) {
    const size_t smem = (size_t)(SG_ROWS * d + SG_KEYS * (d + 1) + SG_KEYS * d) * sizeof(float) +
                        SG_KEYS * sizeof(int);
    static size_t raised = 0;   // the most asked for so far (head sizes differ)
    if (smem > 48 * 1024 && smem > raised) {
        if (cudaFuncSetAttribute(sigmoid_attention_kernel<T, NC>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = smem;
    }
    dim3 grid(num_seqs * tiles_per_seq, n_kv, num_splits);
    MB_LAUNCH((sigmoid_attention_kernel<T, NC>), grid, SG_WARPS * 32, smem, s, (const T*)q,
              (const T*)k_pages, (const T*)v_pages, table, max_pages, q_start, kv_len, head_bias,
              (T*)out, part, n_q, n_kv, d, page_size, scale, window, keep_first, tiles_per_seq,
              num_splits);
    return launch_status();
}

// ---- prompt portions in bfloat16 on the tensor cores ------------------------------------------
// The same sum for head sizes 64 and 128 with mma.sync m16n8k16: a block of NWARPS warps takes
// NWARPS * 16 rows (a warp 16 of them, a thread rows g and g + 8 of those), keys are walked in
// tiles of 64 that cp.async brings into two stages (16-byte pieces, XOR-swizzled by the row),
// S = Q K^T accumulates in float32, the sigmoid of every seen score is taken in float32 and
// rounded to bfloat16 as the A operand of O += P V (values read transposed by ldmatrix). There
// is no running maximum, no rescaling and no denominator. Tiles: those of the kept first
// tokens, then those of the rows' windows, no tile twice.
constexpr int SGM_BN = 64;

template <int D, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
sigmoid_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                             const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ table,
                             int max_pages, const int* __restrict__ q_start,
                             const int* __restrict__ kv_len_of, const float* __restrict__ head_bias,
                             __nv_bfloat16* __restrict__ out, float* __restrict__ part, int n_q, int n_kv,
                             int page_size, float scale, int window, int keep_first, int tiles_per_seq,
                             int num_splits) {
    grid_dependency_sync();
    constexpr int ROWS = NWARPS * 16;
    constexpr int CH = D / 8;        // 16-byte pieces per row
    constexpr int THREADS = NWARPS * 32;
    extern __shared__ __align__(128) unsigned char sgm_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(sgm_raw);   // [ROWS][D]
    __nv_bfloat16* k_s = q_s + ROWS * D;                              // [2][SGM_BN][D]
    __nv_bfloat16* v_s = k_s + 2 * SGM_BN * D;                        // [2][SGM_BN][D]

    const int seq = blockIdx.x / tiles_per_seq;
    const int tile = tiles_per_seq - 1 - (blockIdx.x - seq * tiles_per_seq);
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int group = n_q / n_kv;
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    const int row0 = tile * ROWS;
    if (row0 >= q_len * group) return;
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int idx = tid; idx < ROWS * CH; idx += THREADS) {
        const int r = idx / CH, c = idx - r * CH;
        const int row = row0 + r;
        const int tok = row / group, hg = row - tok * group;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (tok < q_len)
            val = *reinterpret_cast<const uint4*>(q + ((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * D +
                                                  c * 8);
        *reinterpret_cast<uint4*>(q_s + r * D + ((c ^ (r & 7)) * 8)) = val;
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = ks * 2 + (lane >> 4);
        ldmatrix_x4(qf[ks], q_s + r * D + ((c ^ (r & 7)) * 8));
    }

    const int g = lane >> 2, t4 = lane & 3;
    int pos[2];
    bool row_ok[2];
    float bias2[2];                       // the head's number in units of log2(e)
    constexpr float LOG2E = 1.4426950408889634f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row0 + warp * 16 + g + h * 8;
        const int tok = row / group, hg = row - tok * group;
        row_ok[h] = tok < q_len;
        pos[h] = first_pos + tok;
        bias2[h] = head_bias[kvh * group + hg] * LOG2E;
    }
    const int wrow0 = row0 + warp * 16;
    const bool warp_rows_ok = (wrow0 + 15) / group < q_len;
    const int warp_pos_min = first_pos + wrow0 / group;
    const int warp_pos_max = first_pos + (wrow0 + 15) / group;

    // the key tiles of this block: [0, head_hi) for the kept first tokens, [t_lo, t_hi) for the
    // windows; walked as one list with the overlap dropped
    const int tok_min = row0 / group;
    int tok_max = (row0 + ROWS - 1) / group;
    if (tok_max > q_len - 1) tok_max = q_len - 1;
    const int p_min = first_pos + tok_min, p_max = first_pos + tok_max;
    const int t_hi = p_max / SGM_BN + 1;
    int t_lo = 0;
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / SGM_BN;
    int head_hi = 0;
    if (window > 0 && keep_first > 0) head_hi = (keep_first + SGM_BN - 1) / SGM_BN;
    if (head_hi > t_lo) head_hi = t_lo;
    const int count = head_hi + (t_hi - t_lo);
    int n_lo = 0, n_hi = count;
    if (num_splits > 1) {
        const int per = (count + num_splits - 1) / num_splits;
        n_lo = split * per;
        n_hi = n_lo + per < count ? n_lo + per : count;
    }
    auto tile_of = [&](int n) { return n < head_hi ? n : t_lo + (n - head_hi); };

    auto load_tile = [&](int stage, int kt) {
        __nv_bfloat16* kd = k_s + stage * SGM_BN * D;
        __nv_bfloat16* vd = v_s + stage * SGM_BN * D;
        for (int idx = tid; idx < SGM_BN * CH; idx += THREADS) {
            const int j = idx / CH, c = idx - j * CH;
            const int key = kt * SGM_BN + j;
            int page = -1;
            if (key < kv_len) page = table_page(table, seq, max_pages, key / page_size);
            const bool valid = page >= 0;
            const int64_t at =
                valid ? (((int64_t)page * n_kv + kvh) * page_size + (key % page_size)) * D + c * 8 : 0;
            const int sw = (c ^ (j & 7)) * 8;
            cp_async_16(kd + j * D + sw, k_pages + at, valid);
            cp_async_16(vd + j * D + sw, v_pages + at, valid);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const float scale2 = scale * LOG2E;

    if (n_lo < n_hi) load_tile(0, tile_of(n_lo));
    for (int n = n_lo; n < n_hi; ++n) {
        const int kt = tile_of(n);
        const int stage = (n - n_lo) & 1;
        if (n + 1 < n_hi) {
            load_tile(stage ^ 1, tile_of(n + 1));
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const __nv_bfloat16* kt_s = k_s + stage * SGM_BN * D;
        const __nv_bfloat16* vt_s = v_s + stage * SGM_BN * D;

        float s[SGM_BN / 8][4];
#pragma unroll
        for (int i = 0; i < SGM_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < SGM_BN / 16; ++n2) {
                uint32_t b[4];
                const int j = n2 * 16 + (lane & 7) + (lane >> 4) * 8;
                const int c = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(b, kt_s + j * D + ((c ^ (j & 7)) * 8));
                mma_bf16(s[2 * n2], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * n2 + 1], qf[ks], b[2], b[3]);
            }
        }

        // sigmoid(x) = 1 / (1 + 2^(-x log2 e)), float32; an unseen key weighs nothing. A tile
        // that every row of the warp sees whole needs no test per element.
        const int tile_first = kt * SGM_BN, tile_last = tile_first + SGM_BN - 1;
        const bool whole = warp_rows_ok && tile_last <= warp_pos_min && tile_last < kv_len &&
                           (window <= 0 || tile_first > warp_pos_max - window || tile_last < keep_first);
#pragma unroll
        for (int nt = 0; nt < SGM_BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                bool seen = true;
                if (!whole) {
                    const int key = tile_first + nt * 8 + 2 * t4 + (e & 1);
                    seen = row_ok[h] && key <= pos[h] && key < kv_len;
                    if (window > 0) seen = seen && (key > pos[h] - window || key < keep_first);
                }
                const float x2 = fmaf(s[nt][e], scale2, bias2[h]);
                s[nt][e] = seen ? __fdividef(1.f, 1.f + fast_exp2(-x2)) : 0.f;
            }
        }

        // O += P V
#pragma unroll
        for (int kk = 0; kk < SGM_BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < D / 16; ++d2) {
                uint32_t b[4];
                const int j = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = d2 * 2 + (lane >> 4);
                ldmatrix_x4_trans(b, vt_s + j * D + ((c ^ (j & 7)) * 8));
                mma_bf16(o[2 * d2], a, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();  // everyone is done with this stage before it is refilled
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!row_ok[h]) continue;
        const int row = row0 + warp * 16 + g + h * 8;
        const int tok = row / group, hg = row - tok * group;
        const int64_t flat = (int64_t)(q_begin + tok) * n_q + kvh * group + hg;
        if (num_splits == 1) {
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                __nv_bfloat162 v = __floats2bfloat162_rn(o[i][2 * h], o[i][2 * h + 1]);
                *reinterpret_cast<__nv_bfloat162*>(out + flat * D + i * 8 + 2 * t4) = v;
            }
        } else {
            const int64_t at = flat * num_splits + split;
#pragma unroll
            for (int i = 0; i < D / 8; ++i)
                *reinterpret_cast<float2*>(part + at * D + i * 8 + 2 * t4) =
                    make_float2(o[i][2 * h], o[i][2 * h + 1]);
        }
    }
}

template <int D, int NWARPS>
int launch_sigmoid_mma(const void* q, const void* k_pages, const void* v_pages, const int* table,
                       int max_pages, const int* q_start, const int* kv_len, const float* head_bias,
                       void* out, float* part, int n_q, int n_kv, int page_size, float scale, int window,
                       int keep_first, int num_seqs, int tiles_per_seq, int num_splits, cudaStream_t s) {
    typedef __nv_bfloat16 bf;
    const size_t smem = (size_t)(NWARPS * 16 + 4 * SGM_BN) * D * sizeof(bf);
    static bool raised = false;
    if (smem > 40 * 1024 && !raised) {
        if (cudaFuncSetAttribute(sigmoid_attention_mma_kernel<D, NWARPS>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    dim3 grid(num_seqs * tiles_per_seq, n_kv, num_splits);
    MB_LAUNCH((sigmoid_attention_mma_kernel<D, NWARPS>), grid, NWARPS * 32, smem, s, (const bf*)q,
              (const bf*)k_pages, (const bf*)v_pages, table, max_pages, q_start, kv_len, head_bias,
              (bf*)out, part, n_q, n_kv, page_size, scale, window, keep_first, tiles_per_seq,
              num_splits);
    return launch_status();
}

template <typename T>
int dispatch_sigmoid(int nc, const void* q, const void* k_pages, const void* v_pages,
                     const int* table, int max_pages, const int* q_start, const int* kv_len,
                     const float* head_bias, void* out, float* part, int n_q, int n_kv, int d,
                     int page_size, float scale, int window, int keep_first, int num_seqs,
                     int tiles_per_seq, int num_splits, cudaStream_t s) {
#define MB_SG_CASE(N)                                                                             \
    case N:                                                                                       \
        return launch_sigmoid<T, N>(q, k_pages, v_pages, table, max_pages, q_start, kv_len,       \
                                    head_bias, out, part, n_q, n_kv, d, page_size, scale, window, \
                                    keep_first, num_seqs, tiles_per_seq, num_splits, s)
    switch (nc) {
        MB_SG_CASE(1);
        MB_SG_CASE(2);
        MB_SG_CASE(3);
        MB_SG_CASE(4);
        MB_SG_CASE(6);
        MB_SG_CASE(8);
    }
#undef MB_SG_CASE
    return MB_ERR_UNSUPPORTED_SIZE;
}

}  // namespace mb

using namespace mb;

// dtype: the type of q_out and of the pages. wq / wk: float32 norm weights of d numbers, or
// null (no norm). cos_t / sin_t: [positions][rot_dim / 2] float32 (null when rot_dim is 0).
MB_EXPORT int mb_qk_norm_rope_store(const float* pre, int ld, const float* wq, const float* wk,
                                    float eps, const float* cos_t, const float* sin_t, int rot_dim,
                                    int interleaved, const int* positions, const int* seq_of_token,
                                    const int* table, int max_pages, void* k_pages, void* v_pages,
                                    void* q_out, int n_q, int n_kv, int d, int dv,
                                    int values_are_keys, int page_size, int tokens, int dtype,
                                    void* stream) {
    if (tokens <= 0) return MB_OK;
    if (n_q <= 0 || n_kv <= 0 || d <= 0 || dv <= 0 || page_size <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    if (rot_dim < 0 || (rot_dim & 1) || rot_dim > d || (rot_dim > 0 && (!cos_t || !sin_t)))
        return MB_ERR_UNSUPPORTED_SIZE;
    if (values_are_keys && dv != d) return MB_ERR_UNSUPPORTED_SIZE;
    if ((wq == nullptr) != (wk == nullptr)) return MB_ERR_UNSUPPORTED_SIZE;
    const long long warps = (long long)tokens * (n_q + n_kv + (values_are_keys ? 0 : n_kv));
    const long long blocks = (warps + 7) / 8;
    if (blocks > 0x7fffffffLL) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((qk_norm_rope_store_kernel<float>), (int)blocks, 256, 0, s, pre, ld, wq, wk, eps, cos_t,
                  sin_t, rot_dim, interleaved, positions, seq_of_token, table, max_pages,
                  (float*)k_pages, (float*)v_pages, (float*)q_out, n_q, n_kv, d, dv, values_are_keys,
                  page_size, tokens);
    else if (dtype == MB_BF16)
        MB_LAUNCH((qk_norm_rope_store_kernel<__nv_bfloat16>), (int)blocks, 256, 0, s, pre, ld, wq, wk, eps,
                  cos_t, sin_t, rot_dim, interleaved, positions, seq_of_token, table, max_pages,
                  (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out, n_q, n_kv, d,
                  dv, values_are_keys, page_size, tokens);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

MB_EXPORT long long mb_sigmoid_attention_scratch_floats(int tokens, int n_q, int d, int num_splits) {
    return num_splits <= 1 ? 0 : (long long)tokens * n_q * num_splits * d;
}

// q: [tokens][n_q * d] behind norm and rotation; keys and values of size d in the pages. Head
// sizes up to 256. scratch: mb_sigmoid_attention_scratch_floats() floats when num_splits > 1.
MB_EXPORT int mb_sigmoid_attention(const void* q, const void* k_pages, const void* v_pages,
                                   const int* table, int max_pages, const int* q_start,
                                   const int* kv_len, const int* seq_of_token,
                                   const float* head_bias, void* out, float* scratch,
                                   long long scratch_floats, int tokens, int num_seqs, int max_q_len,
                                   int n_q, int n_kv, int d, int page_size, float scale, int window,
                                   int keep_first, int num_splits, int dtype, void* stream) {
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (d <= 0 || d > 256 || n_kv <= 0 || n_q % n_kv) return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || window < 0 || keep_first < 0) return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits < 1) num_splits = 1;
    if (n_kv > 65535 || num_splits > 65535 || n_q > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits > 1 &&
        (!scratch || scratch_floats < mb_sigmoid_attention_scratch_floats(tokens, n_q, d, num_splits)))
        return MB_ERR_SCRATCH;
    const int group = n_q / n_kv;
    const int tiles_per_seq = (max_q_len * group + SG_ROWS - 1) / SG_ROWS;
    int nc = (d + 31) / 32;
    if (nc == 5) nc = 6;
    if (nc == 7) nc = 8;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (dtype == MB_F32)
        rc = dispatch_sigmoid<float>(nc, q, k_pages, v_pages, table, max_pages, q_start, kv_len,
                                     head_bias, out, scratch, n_q, n_kv, d, page_size, scale, window,
                                     keep_first, num_seqs, tiles_per_seq, num_splits, s);
    else if (dtype == MB_BF16)
        rc = dispatch_sigmoid<__nv_bfloat16>(nc, q, k_pages, v_pages, table, max_pages, q_start, kv_len,
                                             head_bias, out, scratch, n_q, n_kv, d, page_size, scale,
                                             window, keep_first, num_seqs, tiles_per_seq, num_splits, s);
    else
        return MB_ERR_BAD_DTYPE;
    if (rc != MB_OK || num_splits == 1) return rc;
    dim3 grid(tokens, n_q);
    if (dtype == MB_F32)
        MB_LAUNCH((sigmoid_attention_sum_kernel<float>), grid, 64, 0, s, scratch, seq_of_token, (float*)out,
                  n_q, d, num_splits);
    else
        MB_LAUNCH((sigmoid_attention_sum_kernel<__nv_bfloat16>), grid, 64, 0, s, scratch, seq_of_token,
                  (__nv_bfloat16*)out, n_q, d, num_splits);
    return launch_status();
}

MB_EXPORT int mb_sigmoid_attention_mma_supports(int d) { return d == 64 || d == 128; }

// The tensor-core kernel: bfloat16, head sizes 64 and 128; everything else as above. A row
// tile is 64 rows (four warps).
MB_EXPORT int mb_sigmoid_attention_mma(const void* q, const void* k_pages, const void* v_pages,
                                       const int* table, int max_pages, const int* q_start,
                                       const int* kv_len, const int* seq_of_token,
                                       const float* head_bias, void* out, float* scratch,
                                       long long scratch_floats, int tokens, int num_seqs,
                                       int max_q_len, int n_q, int n_kv, int d, int page_size,
                                       float scale, int window, int keep_first, int num_splits,
                                       void* stream) {
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (!mb_sigmoid_attention_mma_supports(d) || n_kv <= 0 || n_q % n_kv) return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || window < 0 || keep_first < 0) return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits < 1) num_splits = 1;
    if (n_kv > 65535 || num_splits > 65535 || n_q > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits > 1 &&
        (!scratch || scratch_floats < mb_sigmoid_attention_scratch_floats(tokens, n_q, d, num_splits)))
        return MB_ERR_SCRATCH;
    const int group = n_q / n_kv;
    const int tiles_per_seq = (max_q_len * group + 63) / 64;
    cudaStream_t s = (cudaStream_t)stream;
    const int rc = d == 64
        ? launch_sigmoid_mma<64, 4>(q, k_pages, v_pages, table, max_pages, q_start, kv_len, head_bias, out,
                                    scratch, n_q, n_kv, page_size, scale, window, keep_first, num_seqs,
                                    tiles_per_seq, num_splits, s)
        : launch_sigmoid_mma<128, 4>(q, k_pages, v_pages, table, max_pages, q_start, kv_len, head_bias, out,
                                     scratch, n_q, n_kv, page_size, scale, window, keep_first, num_seqs,
                                     tiles_per_seq, num_splits, s);
    if (rc != MB_OK || num_splits == 1) return rc;
    dim3 grid(tokens, n_q);
    MB_LAUNCH((sigmoid_attention_sum_kernel<__nv_bfloat16>), grid, 64, 0, s, scratch, seq_of_token,
              (__nv_bfloat16*)out, n_q, d, num_splits);
    return launch_status();
}
