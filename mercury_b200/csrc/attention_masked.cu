// Softmax attention over the paged cache under a mask that is a parameter, with the options
// that go with it: a tanh cap on the scores, a sink per head in the denominator, value heads
// of another size than the key heads, and two softmax maps per head whose outputs are
// subtracted (differential attention).
//
// Which keys position p sees: j <= p and (j >= lo(p) or j < keep_first), with
//   lo(p) = 0                         (every key),
//   lo(p) = p - size + 1              (a sliding window of `size` keys), or
//   lo(p) = floor(p / size) * size    (chunks of `size` positions, counted from position 0).
// keep_first: first tokens that stay visible, at their true positions, beside a window.
// score = q . k * scale, then cap * tanh(score / cap) when cap > 0. With sinks the
// denominator of head h also holds exp(sink_h), which has no key and no value.
// With two maps a query head is [q1 | q2] and a key head [k1 | k2] (d numbers each); both maps
// weigh the same values, and the head's output is (a1 - lambda a2) divided by its root mean
// square over the value size (eps inside the root) times out_scale.
//
// In front of it, masked_prepare_kernel: an optional RMS norm over ALL rows of q (and of k) at
// once with a weight per row, the rotation of the first rot_dim numbers of every map of every
// head (halves or neighbours paired), q into the activation buffer, keys and values into
// the pages; the values may be the keys as projected (before norm and rotation).
//
// masked_attention_kernel (CUDA cores, float32 or bfloat16 storage, float32 arithmetic with
// true expf and tanhf): the (token, head of the group) pairs of one sequence and one KV head
// are rows, a block of 8 warps takes 16 of them, keys are walked in tiles of 32 aligned to
// absolute positions, one key per lane for the scores and 32 value features per lane for the
// weighted sum; a block walks the tiles of the kept first tokens and then those from its
// rows' lowest lo on (no tile twice). With num_splits > 1 the tiles are dealt over gridDim.z
// and a second kernel merges the parts in a fixed order.
//
// masked_attention_mma_kernel (bfloat16, prompt portions): the same on mma.sync m16n8k16 for
// d and dv of 64 or 128, 64 rows a block, key tiles of 64 by cp.async in two stages, scores and
// softmax in float32, the weights rounded to bfloat16 as the A operand of the second product.
#include "common.cuh"
#include "mma_sync.cuh"

namespace mb {

constexpr int MK_ROWS = 16;
constexpr int MK_WARPS = 8;
constexpr int MK_RPW = MK_ROWS / MK_WARPS;
constexpr int MK_KEYS = 32;

__device__ __forceinline__ int mask_lo(int kind, int size, int pos) {
    if (kind == 1) return pos - size + 1;
    if (kind == 2) return (pos / size) * size;
    return 0;
}

// pre: [tokens][ld] float32 = [q (n_q * maps * d) | k (n_kv * maps * d) | v (n_kv * dv), unless
// the values are the keys]. One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
masked_prepare_kernel(const float* __restrict__ pre, int ld, const float* __restrict__ wq,
                      const float* __restrict__ wk, float eps, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int rot_dim, int interleaved,
                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      const int* __restrict__ table, int max_pages, T* __restrict__ k_pages,
                      T* __restrict__ v_pages, T* __restrict__ q_out, int n_q, int n_kv, int maps,
                      int d, int dv, int values_are_keys, int page_size) {
    grid_dependency_sync();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    const int qw = n_q * maps * d, kw = n_kv * maps * d;
    const int seq = seq_of_token[t];
    if (seq < 0) {
        for (int c = tid; c < qw; c += blockDim.x) q_out[(int64_t)t * qw + c] = from_float<T>(0.f);
        return;
    }
    const int pos = positions[t];
    const float* row = pre + (int64_t)t * ld;
    float rq = 1.f, rk = 1.f;
    if (wq != nullptr) {
        float sq = 0.f, sk = 0.f;
        for (int c = tid; c < qw; c += blockDim.x) sq = fmaf(row[c], row[c], sq);
        for (int c = tid; c < kw; c += blockDim.x) sk = fmaf(row[qw + c], row[qw + c], sk);
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        rq = 1.f / sqrtf(sq / (float)qw + eps);
        rk = 1.f / sqrtf(sk / (float)kw + eps);
    }
    const int page = table_page(table, seq, max_pages, pos / page_size);
    const int64_t slot = page < 0 ? 0 : ((int64_t)page * n_kv) * page_size + (pos % page_size);
    const int pairs = rot_dim / 2, at_pos = checked_position(pos);
    const int q_units = n_q * maps, units = q_units + n_kv * maps;
    for (int u = warp; u < units; u += warps) {
        const bool is_q = u < q_units;
        const int ku = u - q_units;
        const float* x = row + (is_q ? u * d : qw + ku * d);
        const float* w = wq == nullptr ? nullptr : (is_q ? wq + u * d : wk + ku * d);
        const float rstd = is_q ? rq : rk;
        T* to;
        if (is_q) {
            to = q_out + (int64_t)t * qw + u * d;
        } else {
            if (page < 0) continue;
            const int kvh = ku / maps, map = ku - kvh * maps;
            to = k_pages + (slot + (int64_t)kvh * page_size) * (maps * d) + map * d;
        }
        for (int i = lane; i < pairs; i += 32) {
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + pairs;
            float p = x[a], r = x[b];
            if (w != nullptr) {
                p *= rstd * w[a];
                r *= rstd * w[b];
            }
            const float c = cos_t[(int64_t)at_pos * pairs + i], s = sin_t[(int64_t)at_pos * pairs + i];
            to[a] = from_float<T>(p * c - r * s);
            to[b] = from_float<T>(r * c + p * s);
        }
        for (int c = rot_dim + lane; c < d; c += 32)
            to[c] = from_float<T>(w != nullptr ? x[c] * rstd * w[c] : x[c]);
    }
    if (page < 0) return;
    const float* vx = row + qw + (values_are_keys ? 0 : kw);
    for (int c = tid; c < n_kv * dv; c += blockDim.x) {
        const int kvh = c / dv, i = c - kvh * dv;
        v_pages[(slot + (int64_t)kvh * page_size) * dv + i] = from_float<T>(vx[c]);
    }
}

// What a row knows of its softmax so far, per map.
struct RowSoftmax {
    float m, l;
};

template <typename T, int NC, int MAPS>
__global__ void __launch_bounds__(MK_WARPS * 32)
masked_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const int* __restrict__ table, int max_pages,
                        const int* __restrict__ q_start, const int* __restrict__ kv_len_of,
                        const float* __restrict__ sinks, T* __restrict__ out,
                        float* __restrict__ part_acc, float* __restrict__ part_ml, int n_q, int n_kv,
                        int d, int dv, int page_size, float scale, float cap, int mask_kind,
                        int mask_size, int keep_first, float lambda, float sub_eps, float out_scale,
                        int tiles_per_seq, int num_splits) {
    grid_dependency_sync();
    extern __shared__ float smem[];
    const int seq = blockIdx.x / tiles_per_seq;
    const int tile = blockIdx.x - seq * tiles_per_seq;
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    const int group = n_q / n_kv;
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    const int row0 = tile * MK_ROWS;
    if (row0 >= q_len * group) return;
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;
    const int dk = MAPS * d;

    float* q_s = smem;                                   // [MK_ROWS][dk]
    float* k_s = q_s + MK_ROWS * dk;                     // [MK_KEYS][dk + 1]
    float* v_s = k_s + MK_KEYS * (dk + 1);               // [MK_KEYS][dv]
    int* page_s = reinterpret_cast<int*>(v_s + MK_KEYS * dv);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int idx = tid; idx < MK_ROWS * dk; idx += blockDim.x) {
        const int r = idx / dk, c = idx - r * dk;
        const int row = row0 + r;
        const int tok = row / group, hg = row - tok * group;
        q_s[idx] = tok < q_len ? to_float(q[((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * dk + c]) : 0.f;
    }
    int row_pos[MK_RPW], row_lo[MK_RPW];
    bool row_ok[MK_RPW];
#pragma unroll
    for (int rr = 0; rr < MK_RPW; ++rr) {
        const int row = row0 + warp * MK_RPW + rr;
        const int tok = row / group;
        row_ok[rr] = tok < q_len;
        row_pos[rr] = first_pos + tok;
        row_lo[rr] = mask_lo(mask_kind, mask_size, row_pos[rr]);
    }
    // the key tiles of this block: [0, head_hi) for the kept first tokens, [t_lo, t_hi) from
    // the lowest lo of its rows on; walked as one list with the overlap dropped
    const int tok_min = row0 / group;
    int tok_max = (row0 + MK_ROWS - 1) / group;
    if (tok_max > q_len - 1) tok_max = q_len - 1;
    const int p_min = first_pos + tok_min, p_max = first_pos + tok_max;
    const int t_hi = p_max / MK_KEYS + 1;
    const int lo_min = mask_lo(mask_kind, mask_size, p_min);
    const int t_lo = lo_min > 0 ? lo_min / MK_KEYS : 0;
    int head_hi = keep_first > 0 ? (keep_first + MK_KEYS - 1) / MK_KEYS : 0;
    if (head_hi > t_lo) head_hi = t_lo;
    const int count = head_hi + (t_hi - t_lo);
    int n_lo = 0, n_hi = count;
    if (num_splits > 1) {
        const int per = (count + num_splits - 1) / num_splits;
        n_lo = split * per;
        n_hi = n_lo + per < count ? n_lo + per : count;
    }

    float acc[MK_RPW][MAPS][NC];
    RowSoftmax st[MK_RPW][MAPS];
#pragma unroll
    for (int rr = 0; rr < MK_RPW; ++rr)
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            st[rr][mp].m = -INFINITY;
            st[rr][mp].l = 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[rr][mp][c] = 0.f;
        }

    for (int n = n_lo; n < n_hi; ++n) {
        const int kt = n < head_hi ? n : t_lo + (n - head_hi);
        __syncthreads();
        if (tid < MK_KEYS) {
            const int key = kt * MK_KEYS + tid;
            int page = -1;
            if (key < kv_len) page = table_page(table, seq, max_pages, key / page_size);
            page_s[tid] = page;
        }
        __syncthreads();
        {
            // eight threads a key: the page and the slot are looked up once, no division a number
            const int j = tid >> 3, sub = tid & 7;
            const int page = page_s[j];
            const int key = kt * MK_KEYS + j;
            const int64_t at = page >= 0 ? ((int64_t)page * n_kv + kvh) * page_size + (key % page_size) : 0;
            const T* kp = k_pages + at * dk;
            const T* vp = v_pages + at * dv;
            for (int c = sub; c < dk; c += 8) k_s[j * (dk + 1) + c] = page >= 0 ? to_float(kp[c]) : 0.f;
            for (int c = sub; c < dv; c += 8) v_s[j * dv + c] = page >= 0 ? to_float(vp[c]) : 0.f;
        }
        __syncthreads();
        const int key = kt * MK_KEYS + lane;
        const bool key_ok = page_s[lane] >= 0;
        const float* krow = k_s + lane * (dk + 1);
#pragma unroll
        for (int rr = 0; rr < MK_RPW; ++rr) {
            const bool seen = row_ok[rr] && key_ok && key <= row_pos[rr] &&
                              (key >= row_lo[rr] || key < keep_first);
            if (__ballot_sync(0xffffffffu, seen) == 0u) continue;
            const float* qrow = q_s + (warp * MK_RPW + rr) * dk;
#pragma unroll
            for (int mp = 0; mp < MAPS; ++mp) {
                float s = 0.f;
                for (int c = 0; c < d; ++c) s = fmaf(qrow[mp * d + c], krow[mp * d + c], s);
                s *= scale;
                if (cap > 0.f) s = cap * tanhf(s / cap);
                if (!seen) s = -INFINITY;
                const float m_new = fmaxf(st[rr][mp].m, warp_max(s));
                const float corr = expf(st[rr][mp].m - m_new);      // exp(-inf) = 0 at the start
                const float p = seen ? expf(s - m_new) : 0.f;
                st[rr][mp].l = st[rr][mp].l * corr + warp_sum(p);
                st[rr][mp].m = m_new;
#pragma unroll
                for (int c = 0; c < NC; ++c) acc[rr][mp][c] *= corr;
#pragma unroll 4
                for (int j = 0; j < MK_KEYS; ++j) {
                    const float pj = __shfl_sync(0xffffffffu, p, j);
                    if (pj == 0.f) continue;
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        const int dim = lane + 32 * c;
                        if (dim < dv) acc[rr][mp][c] = fmaf(pj, v_s[j * dv + dim], acc[rr][mp][c]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int rr = 0; rr < MK_RPW; ++rr) {
        if (!row_ok[rr]) continue;
        const int row = row0 + warp * MK_RPW + rr;
        const int tok = row / group, hg = row - tok * group;
        const int head = kvh * group + hg;
        const int64_t flat = (int64_t)(q_begin + tok) * n_q + head;
        if (num_splits > 1) {
#pragma unroll
            for (int mp = 0; mp < MAPS; ++mp) {
                const int64_t at = (flat * num_splits + split) * MAPS + mp;
                if (lane == 0) {
                    part_ml[at * 2] = st[rr][mp].m;
                    part_ml[at * 2 + 1] = st[rr][mp].l;
                }
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int dim = lane + 32 * c;
                    if (dim < dv) part_acc[at * dv + dim] = acc[rr][mp][c];
                }
            }
            continue;
        }
        float o[NC];
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            float m = st[rr][mp].m, l = st[rr][mp].l, keep = 1.f;
            if (sinks != nullptr) {
                const float sk = sinks[head];
                const float m2 = fmaxf(m, sk);
                keep = expf(m - m2);
                l = l * keep + expf(sk - m2);
            }
            const float inv = l > 0.f ? keep / l : 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float a = acc[rr][mp][c] * inv;
                o[c] = mp == 0 ? a : o[c] - lambda * a;
            }
        }
        if (MAPS == 2) {
            float ss = 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if (lane + 32 * c < dv) ss = fmaf(o[c], o[c], ss);
            ss = warp_sum(ss);
            const float r = out_scale / sqrtf(ss / (float)dv + sub_eps);
#pragma unroll
            for (int c = 0; c < NC; ++c) o[c] *= r;
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int dim = lane + 32 * c;
            if (dim < dv) out[flat * dv + dim] = from_float<T>(o[c]);
        }
    }
}

// The parts of a (token, head) merged, split 0 first: per map the largest maximum (the sink's
// number included), the sums and the weighted values brought to it; then, with two maps,
// their difference and its norm. A block per (token, head), a thread per value column: the
// first warp reads the parts' maxima and sums side by side (a lane a part) and leaves a
// weight per part, then every thread adds up its column over the parts, whose reads do not
// wait for one another.
template <typename T, int MAPS>
__global__ void masked_attention_merge_kernel(const float* __restrict__ part_acc,
                                              const float* __restrict__ part_ml,
                                              const int* __restrict__ seq_of_token,
                                              const float* __restrict__ sinks, T* __restrict__ out,
                                              int n_q, int dv, int num_splits, float lambda,
                                              float sub_eps, float out_scale) {
    grid_dependency_sync();
    extern __shared__ float w_s[];          // [MAPS][num_splits] weights, then [MAPS] 1 / sum
    __shared__ float scratch[33];
    float* inv_s = w_s + MAPS * num_splits;
    const int tok = blockIdx.x, head = blockIdx.y;
    const int c = threadIdx.x, lane = c & 31;
    const int64_t flat = (int64_t)tok * n_q + head;
    if (seq_of_token[tok] < 0) {
        if (c < dv) out[flat * dv + c] = from_float<T>(0.f);
        return;
    }
    if (c < 32) {
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            const float sink = sinks != nullptr ? sinks[head] : -INFINITY;
            float m = sink;
            for (int z = lane; z < num_splits; z += 32)
                m = fmaxf(m, part_ml[((flat * num_splits + z) * MAPS + mp) * 2]);
            m = warp_max(m);
            float l = 0.f;
            for (int z = lane; z < num_splits; z += 32) {
                const int64_t at = (flat * num_splits + z) * MAPS + mp;
                const float mz = part_ml[at * 2];
                const float w = mz == -INFINITY ? 0.f : expf(mz - m);
                w_s[mp * num_splits + z] = w;
                l = fmaf(part_ml[at * 2 + 1], w, l);
            }
            l = warp_sum(l);
            if (sinks != nullptr) l += expf(sink - m);
            if (lane == 0) inv_s[mp] = l > 0.f ? 1.f / l : 0.f;
        }
    }
    __syncthreads();
    float o = 0.f;
    if (c < dv) {
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            float a = 0.f;
#pragma unroll 8
            for (int z = 0; z < num_splits; ++z)
                a = fmaf(part_acc[((flat * num_splits + z) * MAPS + mp) * dv + c], w_s[mp * num_splits + z], a);
            a *= inv_s[mp];
            o = mp == 0 ? a : o - lambda * a;
        }
    }
    if (MAPS == 2) {
        const float ss = block_sum(c < dv ? o * o : 0.f, scratch);
        o *= out_scale / sqrtf(ss / (float)dv + sub_eps);
    }
    if (c < dv) out[flat * dv + c] = from_float<T>(o);
}

struct MaskedArgs {
    const void *q, *k_pages, *v_pages;
    const int* table;
    int max_pages;
    const int *q_start, *kv_len, *seq_of_token;
    const float* sinks;
    void* out;
    float *part_acc, *part_ml;
    int tokens, num_seqs, n_q, n_kv, d, dv, page_size;
    float scale, cap;
    int mask_kind, mask_size, keep_first;
    float lambda, sub_eps, out_scale;
    int tiles_per_seq, num_splits;
};

template <typename T, int NC, int MAPS>
int launch_masked(const MaskedArgs& a, cudaStream_t s) {
    const int dk = MAPS * a.d;
    const size_t smem = (size_t)(MK_ROWS * dk + MK_KEYS * (dk + 1) + MK_KEYS * a.dv) * sizeof(float) +
                        MK_KEYS * sizeof(int);
    if (smem > 200 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    static size_t raised = 0;   // the most asked for so far (head sizes differ)
    if (smem > 40 * 1024 && smem > raised) {
        if (cudaFuncSetAttribute(masked_attention_kernel<T, NC, MAPS>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = smem;
    }
    dim3 grid(a.num_seqs * a.tiles_per_seq, a.n_kv, a.num_splits);
    MB_LAUNCH((masked_attention_kernel<T, NC, MAPS>), grid, MK_WARPS * 32, smem, s, (const T*)a.q,
              (const T*)a.k_pages, (const T*)a.v_pages, a.table, a.max_pages, a.q_start, a.kv_len,
              a.sinks, (T*)a.out, a.part_acc, a.part_ml, a.n_q, a.n_kv, a.d, a.dv, a.page_size, a.scale,
              a.cap, a.mask_kind, a.mask_size, a.keep_first, a.lambda, a.sub_eps, a.out_scale,
              a.tiles_per_seq, a.num_splits);
    if (launch_status() != MB_OK) return MB_ERR_LAUNCH;
    if (a.num_splits == 1) return MB_OK;
    dim3 mgrid(a.tokens, a.n_q);
    MB_LAUNCH((masked_attention_merge_kernel<T, MAPS>), mgrid, (a.dv + 31) / 32 * 32,
              (size_t)(MAPS * a.num_splits + MAPS) * sizeof(float), s,
              a.part_acc, a.part_ml, a.seq_of_token, a.sinks, (T*)a.out, a.n_q, a.dv, a.num_splits,
              a.lambda, a.sub_eps, a.out_scale);
    return launch_status();
}

template <typename T, int MAPS>
int dispatch_masked(int nc, const MaskedArgs& a, cudaStream_t s) {
    switch (nc) {
        case 1: return launch_masked<T, 1, MAPS>(a, s);
        case 2: return launch_masked<T, 2, MAPS>(a, s);
        case 4: return launch_masked<T, 4, MAPS>(a, s);
        case 8: return launch_masked<T, 8, MAPS>(a, s);
    }
    return MB_ERR_UNSUPPORTED_SIZE;
}

// ---- prompt portions in bfloat16 on the tensor cores ------------------------------------------
// The same attention for key sizes D and value sizes DV of 64 and 128 with mma.sync m16n8k16: a
// block of NWARPS warps takes NWARPS * 16 rows (a warp 16 of them, a thread rows g and g + 8 of
// those), keys are walked in tiles of 64 that cp.async brings into two stages (16-byte pieces,
// XOR-swizzled by the row; a key row's maps lie in planes of their own), S = Q K^T accumulates
// in float32, cap, mask and softmax run in float32 on the accumulators (base-2 exponentials
// of scores in units of log2 e, a running maximum and sum per row and map), the weights are
// rounded to bfloat16 as the A operand of O += P V (values read transposed by ldmatrix). With
// two maps each has its own accumulators over the same value tile, and the query fragments
// are read from shared memory tile by tile instead of being held in registers.
constexpr int MKM_BN = 64;
constexpr float MK_LOG2E = 1.4426950408889634f;

template <int D, int DV, int MAPS, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
masked_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                            const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ table,
                            int max_pages, const int* __restrict__ q_start,
                            const int* __restrict__ kv_len_of, const float* __restrict__ sinks,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ part_acc,
                            float* __restrict__ part_ml, int n_q, int n_kv, int page_size, float scale,
                            float cap, int mask_kind, int mask_size, int keep_first, float lambda,
                            float sub_eps, float out_scale, int tiles_per_seq, int num_splits) {
    grid_dependency_sync();
    constexpr int ROWS = NWARPS * 16;
    constexpr int CH = D / 8, CHV = DV / 8;        // 16-byte pieces per row
    constexpr int THREADS = NWARPS * 32;
    constexpr int DK = MAPS * D;
    extern __shared__ __align__(128) unsigned char mkm_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(mkm_raw);   // [MAPS][ROWS][D]
    __nv_bfloat16* k_s = q_s + MAPS * ROWS * D;                        // [2][MAPS][MKM_BN][D]
    __nv_bfloat16* v_s = k_s + 2 * MAPS * MKM_BN * D;                  // [2][MKM_BN][DV]

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

    for (int idx = tid; idx < ROWS * MAPS * CH; idx += THREADS) {
        const int r = idx / (MAPS * CH), rest = idx - r * (MAPS * CH);
        const int mp = rest / CH, c = rest - mp * CH;
        const int row = row0 + r;
        const int tok = row / group, hg = row - tok * group;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (tok < q_len)
            val = *reinterpret_cast<const uint4*>(q + ((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * DK +
                                                  mp * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + (mp * ROWS + r) * D + ((c ^ (r & 7)) * 8)) = val;
    }
    __syncthreads();
    uint32_t qf[MAPS == 1 ? D / 16 : 1][4];
    if (MAPS == 1) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int c = ks * 2 + (lane >> 4);
            ldmatrix_x4(qf[MAPS == 1 ? ks : 0], q_s + r * D + ((c ^ (r & 7)) * 8));
        }
    }

    const int g = lane >> 2, t4 = lane & 3;
    int pos[2], lo[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row0 + warp * 16 + g + h * 8;
        const int tok = row / group;
        row_ok[h] = tok < q_len;
        pos[h] = first_pos + tok;
        lo[h] = mask_lo(mask_kind, mask_size, pos[h]);
    }
    const int wrow0 = row0 + warp * 16;
    const bool warp_rows_ok = (wrow0 + 15) / group < q_len;
    const int warp_pos_min = first_pos + wrow0 / group;
    const int warp_pos_max = first_pos + (wrow0 + 15) / group;
    const int warp_lo_max = mask_lo(mask_kind, mask_size, warp_pos_max);

    const int tok_min = row0 / group;
    int tok_max = (row0 + ROWS - 1) / group;
    if (tok_max > q_len - 1) tok_max = q_len - 1;
    const int p_min = first_pos + tok_min, p_max = first_pos + tok_max;
    const int t_hi = p_max / MKM_BN + 1;
    const int lo_min = mask_lo(mask_kind, mask_size, p_min);
    const int t_lo = lo_min > 0 ? lo_min / MKM_BN : 0;
    int head_hi = keep_first > 0 ? (keep_first + MKM_BN - 1) / MKM_BN : 0;
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
        __nv_bfloat16* kd = k_s + stage * MAPS * MKM_BN * D;
        __nv_bfloat16* vd = v_s + stage * MKM_BN * DV;
        for (int idx = tid; idx < MKM_BN * (MAPS * CH + CHV); idx += THREADS) {
            const int j = idx / (MAPS * CH + CHV), c = idx - j * (MAPS * CH + CHV);
            const int key = kt * MKM_BN + j;
            int page = -1;
            if (key < kv_len) page = table_page(table, seq, max_pages, key / page_size);
            const bool valid = page >= 0;
            const int64_t at = valid ? ((int64_t)page * n_kv + kvh) * page_size + (key % page_size) : 0;
            if (c < MAPS * CH) {
                const int mp = c / CH, cc = c - mp * CH;
                cp_async_16(kd + (mp * MKM_BN + j) * D + ((cc ^ (j & 7)) * 8), k_pages + at * DK + c * 8, valid);
            } else {
                const int cc = c - MAPS * CH;
                cp_async_16(vd + j * DV + ((cc ^ (j & 7)) * 8), v_pages + at * DV + cc * 8, valid);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    float o[MAPS][DV / 8][4];
    float m_run[MAPS][2], l_run[MAPS][2];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) o[mp][i][0] = o[mp][i][1] = o[mp][i][2] = o[mp][i][3] = 0.f;
        m_run[mp][0] = m_run[mp][1] = -INFINITY;
        l_run[mp][0] = l_run[mp][1] = 0.f;
    }
    const float scale2 = scale * MK_LOG2E;

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
        const __nv_bfloat16* vt_s = v_s + stage * MKM_BN * DV;
        // a tile that every row of the warp sees whole needs no test per element
        const int tile_first = kt * MKM_BN, tile_last = tile_first + MKM_BN - 1;
        const bool whole = warp_rows_ok && tile_last <= warp_pos_min && tile_last < kv_len &&
                           (tile_first >= warp_lo_max || tile_last < keep_first);
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            const __nv_bfloat16* kt_s = k_s + (stage * MAPS + mp) * MKM_BN * D;
            float s[MKM_BN / 8][4];
#pragma unroll
            for (int i = 0; i < MKM_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a[4];
                if (MAPS == 1) {
                    a[0] = qf[MAPS == 1 ? ks : 0][0], a[1] = qf[MAPS == 1 ? ks : 0][1];
                    a[2] = qf[MAPS == 1 ? ks : 0][2], a[3] = qf[MAPS == 1 ? ks : 0][3];
                } else {
                    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int c = ks * 2 + (lane >> 4);
                    ldmatrix_x4(a, q_s + (mp * ROWS + r) * D + ((c ^ (r & 7)) * 8));
                }
#pragma unroll
                for (int n2 = 0; n2 < MKM_BN / 16; ++n2) {
                    uint32_t b[4];
                    const int j = n2 * 16 + (lane & 7) + (lane >> 4) * 8;
                    const int c = ks * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(b, kt_s + j * D + ((c ^ (j & 7)) * 8));
                    mma_bf16(s[2 * n2], a, b[0], b[1]);
                    mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
                }
            }
            // scores in units of log2 e, capped, unseen keys at -inf; the tile's maximum per row
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < MKM_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    float x2 = s[nt][e] * scale2;
                    if (cap > 0.f) {
                        // cap tanh(x / cap), tanh(y) = 1 - 2 / (2^(2 y log2 e) + 1)
                        const float y2 = x2 * __fdividef(2.f, cap);
                        x2 = cap * MK_LOG2E * (1.f - __fdividef(2.f, fast_exp2(y2) + 1.f));
                    }
                    if (!whole) {
                        const int key = tile_first + nt * 8 + 2 * t4 + (e & 1);
                        const bool seen = row_ok[h] && key <= pos[h] && key < kv_len &&
                                          (key >= lo[h] || key < keep_first);
                        if (!seen) x2 = -INFINITY;
                    }
                    s[nt][e] = x2;
                    tmax[h] = fmaxf(tmax[h], x2);
                }
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                const float m_new = fmaxf(m_run[mp][h], tmax[h]);
                m_use[h] = m_new == -INFINITY ? 0.f : m_new;
                corr[h] = fast_exp2(m_run[mp][h] - m_use[h]);
                m_run[mp][h] = m_new;
                l_run[mp][h] *= corr[h];
            }
#pragma unroll
            for (int nt = 0; nt < MKM_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = fast_exp2(s[nt][e] - m_use[e >> 1]);
                    s[nt][e] = p;
                    l_run[mp][e >> 1] += p;
                }
            }
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                o[mp][i][0] *= corr[0];
                o[mp][i][1] *= corr[0];
                o[mp][i][2] *= corr[1];
                o[mp][i][3] *= corr[1];
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < MKM_BN / 16; ++kk) {
                uint32_t a[4];
                a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int d2 = 0; d2 < DV / 16; ++d2) {
                    uint32_t b[4];
                    const int j = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int c = d2 * 2 + (lane >> 4);
                    ldmatrix_x4_trans(b, vt_s + j * DV + ((c ^ (j & 7)) * 8));
                    mma_bf16(o[mp][2 * d2], a, b[0], b[1]);
                    mma_bf16(o[mp][2 * d2 + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();  // everyone is done with this stage before it is refilled
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row0 + warp * 16 + g + h * 8;
        const int tok = row / group, hg = row - tok * group;
        const int head = kvh * group + hg;
        const int64_t flat = (int64_t)(q_begin + tok) * n_q + head;
        float inv[MAPS];
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            float l = l_run[mp][h];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            l_run[mp][h] = l;
            float keep = 1.f;
            if (num_splits == 1 && sinks != nullptr && row_ok[h]) {
                const float sk = sinks[head] * MK_LOG2E;
                const float m2 = fmaxf(m_run[mp][h], sk);
                keep = fast_exp2(m_run[mp][h] - m2);
                l = l * keep + fast_exp2(sk - m2);
            }
            inv[mp] = l > 0.f ? keep / l : 0.f;
        }
        if (num_splits > 1) {
            if (!row_ok[h]) continue;
#pragma unroll
            for (int mp = 0; mp < MAPS; ++mp) {
                const int64_t at = (flat * num_splits + split) * MAPS + mp;
                if (t4 == 0) {
                    part_ml[at * 2] = m_run[mp][h] / MK_LOG2E;      // natural units, as the merge takes them
                    part_ml[at * 2 + 1] = l_run[mp][h];
                }
#pragma unroll
                for (int i = 0; i < DV / 8; ++i)
                    *reinterpret_cast<float2*>(part_acc + at * DV + i * 8 + 2 * t4) =
                        make_float2(o[mp][i][2 * h], o[mp][i][2 * h + 1]);
            }
            continue;
        }
        float r = 1.f;
        if (MAPS == 2) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float v = o[0][i][2 * h + e] * inv[0] - lambda * o[MAPS - 1][i][2 * h + e] * inv[MAPS - 1];
                    o[0][i][2 * h + e] = v;
                    ss = fmaf(v, v, ss);
                }
            }
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            r = out_scale / sqrtf(ss / (float)DV + sub_eps);
        } else {
            r = inv[0];
        }
        if (!row_ok[h]) continue;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            __nv_bfloat162 v = __floats2bfloat162_rn(o[0][i][2 * h] * r, o[0][i][2 * h + 1] * r);
            *reinterpret_cast<__nv_bfloat162*>(out + flat * DV + i * 8 + 2 * t4) = v;
        }
    }
}

template <int D, int DV, int MAPS>
int launch_masked_mma(const MaskedArgs& a, cudaStream_t s) {
    typedef __nv_bfloat16 bf;
    constexpr int NWARPS = 4;
    const size_t smem = (size_t)(MAPS * NWARPS * 16 * D + 2 * MAPS * MKM_BN * D + 2 * MKM_BN * DV) * sizeof(bf);
    static bool raised = false;
    if (smem > 40 * 1024 && !raised) {
        if (cudaFuncSetAttribute(masked_attention_mma_kernel<D, DV, MAPS, NWARPS>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    dim3 grid(a.num_seqs * a.tiles_per_seq, a.n_kv, a.num_splits);
    MB_LAUNCH((masked_attention_mma_kernel<D, DV, MAPS, NWARPS>), grid, NWARPS * 32, smem, s, (const bf*)a.q,
              (const bf*)a.k_pages, (const bf*)a.v_pages, a.table, a.max_pages, a.q_start, a.kv_len, a.sinks,
              (bf*)a.out, a.part_acc, a.part_ml, a.n_q, a.n_kv, a.page_size, a.scale, a.cap, a.mask_kind,
              a.mask_size, a.keep_first, a.lambda, a.sub_eps, a.out_scale, a.tiles_per_seq, a.num_splits);
    if (launch_status() != MB_OK) return MB_ERR_LAUNCH;
    if (a.num_splits == 1) return MB_OK;
    dim3 mgrid(a.tokens, a.n_q);
    MB_LAUNCH((masked_attention_merge_kernel<bf, MAPS>), mgrid, DV, (size_t)(MAPS * a.num_splits + MAPS) * sizeof(float), s,
              a.part_acc,
              a.part_ml, a.seq_of_token, a.sinks, (bf*)a.out, a.n_q, DV, a.num_splits, a.lambda, a.sub_eps,
              a.out_scale);
    return launch_status();
}

}  // namespace mb

using namespace mb;

// dtype: the type of q_out and of the pages. wq / wk: float32 norm weights over the whole q
// and k projections (n_q * maps * d and n_kv * maps * d numbers), or null (no norm). cos_t /
// sin_t: [positions][rot_dim / 2] float32 (null when rot_dim is 0).
MB_EXPORT int mb_masked_prepare(const float* pre, int ld, const float* wq, const float* wk, float eps,
                                const float* cos_t, const float* sin_t, int rot_dim, int interleaved,
                                const int* positions, const int* seq_of_token, const int* table,
                                int max_pages, void* k_pages, void* v_pages, void* q_out, int n_q,
                                int n_kv, int maps, int d, int dv, int values_are_keys, int page_size,
                                int tokens, int dtype, void* stream) {
    if (tokens <= 0) return MB_OK;
    if (n_q <= 0 || n_kv <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || maps < 1 || maps > 2)
        return MB_ERR_UNSUPPORTED_SIZE;
    if (rot_dim < 0 || (rot_dim & 1) || rot_dim > d || (rot_dim > 0 && (!cos_t || !sin_t)))
        return MB_ERR_UNSUPPORTED_SIZE;
    if (values_are_keys && dv != maps * d) return MB_ERR_UNSUPPORTED_SIZE;
    if ((wq == nullptr) != (wk == nullptr)) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((masked_prepare_kernel<float>), tokens, 256, 0, s, pre, ld, wq, wk, eps, cos_t, sin_t,
                  rot_dim, interleaved, positions, seq_of_token, table, max_pages, (float*)k_pages,
                  (float*)v_pages, (float*)q_out, n_q, n_kv, maps, d, dv, values_are_keys, page_size);
    else if (dtype == MB_BF16)
        MB_LAUNCH((masked_prepare_kernel<__nv_bfloat16>), tokens, 256, 0, s, pre, ld, wq, wk, eps, cos_t,
                  sin_t, rot_dim, interleaved, positions, seq_of_token, table, max_pages,
                  (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out, n_q, n_kv,
                  maps, d, dv, values_are_keys, page_size);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

// floats of scratch the split form needs: the parts' weighted values, then their (max, sum)
MB_EXPORT long long mb_masked_attention_scratch_floats(int tokens, int n_q, int maps, int dv,
                                                       int num_splits) {
    return num_splits <= 1 ? 0 : (long long)tokens * n_q * num_splits * maps * (dv + 2);
}

// q: [tokens][n_q * maps * d] behind norm and rotation; keys of maps * d numbers and values of
// dv numbers a head in the pages. mask_kind 0: every key, 1: sliding window, 2: chunks.
MB_EXPORT int mb_masked_attention(const void* q, const void* k_pages, const void* v_pages,
                                  const int* table, int max_pages, const int* q_start,
                                  const int* kv_len, const int* seq_of_token, const float* sinks,
                                  void* out, float* scratch, long long scratch_floats, int tokens,
                                  int num_seqs, int max_q_len, int n_q, int n_kv, int maps, int d,
                                  int dv, int page_size, float scale, float cap, int mask_kind,
                                  int mask_size, int keep_first, float lambda, float sub_eps,
                                  float out_scale, int num_splits, int dtype, void* stream) {
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (d <= 0 || dv <= 0 || dv > 256 || n_kv <= 0 || n_q % n_kv || maps < 1 || maps > 2)
        return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || mask_kind < 0 || mask_kind > 2 || keep_first < 0 ||
        (mask_kind != 0 && mask_size <= 0) || (mask_kind != 1 && keep_first != 0))
        return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits < 1) num_splits = 1;
    if (n_kv > 65535 || num_splits > 65535 || n_q > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    const long long need = mb_masked_attention_scratch_floats(tokens, n_q, maps, dv, num_splits);
    if (num_splits > 1 && (!scratch || scratch_floats < need)) return MB_ERR_SCRATCH;
    MaskedArgs a;
    a.q = q, a.k_pages = k_pages, a.v_pages = v_pages, a.table = table, a.max_pages = max_pages;
    a.q_start = q_start, a.kv_len = kv_len, a.seq_of_token = seq_of_token, a.sinks = sinks, a.out = out;
    a.part_acc = scratch;
    a.part_ml = scratch ? scratch + (long long)tokens * n_q * num_splits * maps * dv : nullptr;
    a.tokens = tokens, a.num_seqs = num_seqs, a.n_q = n_q, a.n_kv = n_kv, a.d = d, a.dv = dv;
    a.page_size = page_size, a.scale = scale, a.cap = cap, a.mask_kind = mask_kind;
    a.mask_size = mask_size, a.keep_first = keep_first, a.lambda = lambda, a.sub_eps = sub_eps;
    a.out_scale = out_scale, a.num_splits = num_splits;
    const int group = n_q / n_kv;
    a.tiles_per_seq = (max_q_len * group + MK_ROWS - 1) / MK_ROWS;
    const int nc = dv <= 32 ? 1 : (dv <= 64 ? 2 : (dv <= 128 ? 4 : 8));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        return maps == 1 ? dispatch_masked<float, 1>(nc, a, s) : dispatch_masked<float, 2>(nc, a, s);
    if (dtype == MB_BF16)
        return maps == 1 ? dispatch_masked<__nv_bfloat16, 1>(nc, a, s)
                         : dispatch_masked<__nv_bfloat16, 2>(nc, a, s);
    return MB_ERR_BAD_DTYPE;
}

// What the tensor-core kernel takes: key and value sizes of 64 and 128, two maps with keys of 64.
MB_EXPORT int mb_masked_attention_mma_supports(int maps, int d, int dv) {
    if (dv != 64 && dv != 128) return 0;
    if (maps == 1) return d == 64 || d == 128;
    return maps == 2 && d == 64;
}

// The tensor-core kernel: bfloat16; everything else as mb_masked_attention. A row tile is 64
// rows (four warps).
MB_EXPORT int mb_masked_attention_mma(const void* q, const void* k_pages, const void* v_pages,
                                      const int* table, int max_pages, const int* q_start,
                                      const int* kv_len, const int* seq_of_token, const float* sinks,
                                      void* out, float* scratch, long long scratch_floats, int tokens,
                                      int num_seqs, int max_q_len, int n_q, int n_kv, int maps, int d,
                                      int dv, int page_size, float scale, float cap, int mask_kind,
                                      int mask_size, int keep_first, float lambda, float sub_eps,
                                      float out_scale, int num_splits, void* stream) {
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (!mb_masked_attention_mma_supports(maps, d, dv) || n_kv <= 0 || n_q % n_kv)
        return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || mask_kind < 0 || mask_kind > 2 || keep_first < 0 ||
        (mask_kind != 0 && mask_size <= 0) || (mask_kind != 1 && keep_first != 0))
        return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits < 1) num_splits = 1;
    if (n_kv > 65535 || num_splits > 65535 || n_q > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    const long long need = mb_masked_attention_scratch_floats(tokens, n_q, maps, dv, num_splits);
    if (num_splits > 1 && (!scratch || scratch_floats < need)) return MB_ERR_SCRATCH;
    MaskedArgs a;
    a.q = q, a.k_pages = k_pages, a.v_pages = v_pages, a.table = table, a.max_pages = max_pages;
    a.q_start = q_start, a.kv_len = kv_len, a.seq_of_token = seq_of_token, a.sinks = sinks, a.out = out;
    a.part_acc = scratch;
    a.part_ml = scratch ? scratch + (long long)tokens * n_q * num_splits * maps * dv : nullptr;
    a.tokens = tokens, a.num_seqs = num_seqs, a.n_q = n_q, a.n_kv = n_kv, a.d = d, a.dv = dv;
    a.page_size = page_size, a.scale = scale, a.cap = cap, a.mask_kind = mask_kind;
    a.mask_size = mask_size, a.keep_first = keep_first, a.lambda = lambda, a.sub_eps = sub_eps;
    a.out_scale = out_scale, a.num_splits = num_splits;
    a.tiles_per_seq = (max_q_len * (n_q / n_kv) + 63) / 64;
    cudaStream_t s = (cudaStream_t)stream;
    if (maps == 2) return dv == 64 ? launch_masked_mma<64, 64, 2>(a, s) : launch_masked_mma<64, 128, 2>(a, s);
    if (d == 64) return dv == 64 ? launch_masked_mma<64, 64, 1>(a, s) : launch_masked_mma<64, 128, 1>(a, s);
    return dv == 64 ? launch_masked_mma<128, 64, 1>(a, s) : launch_masked_mma<128, 128, 1>(a, s);
}
