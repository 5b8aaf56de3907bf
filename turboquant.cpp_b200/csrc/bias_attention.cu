// Attention with a learned distance bias, a window that keeps a sequence's first positions, and a sink in the
// softmax's denominator, over a paged cache whose rows hold a key and a value of different sizes.
//
//   score(i, j) = cap(q_i . k_j * scale) + bias[min(i - j, far)][head]   (bias: a table per distance, or none;
//                                                                          cap(s) = softcap * tanh(s / softcap), or s if softcap is 0)
//   i sees j    iff j <= i and (window == 0 or i - j < window or j < keep_first);
//               with cells (cell > 0) instead iff j <= i and floor(i / cell) = floor(j / cell)
//   p_j         = exp(score_j) / (exp(sink[head]) + sum over the visible j of exp(score_j))   (sink: per head, or none)
//   out_i       = sum_j p_j v_j
//
// Query head h reads key/value head h / (heads / kv heads).  Scores, the softmax and the weighted sums are fp32.
// Cache layout of one layer: [page][kv head][slot in page][dk + dv], a position's key followed by its value; a
// sequence's position p lives in page table[seq][p / page_size] at slot p % page_size.
//
//   tq_bias_kv_write       splits a fused projection [q | k | v] (fp32): queries to a buffer, keys and values into the
//                          cache; values may be mixed with another layer's values of the same token,
//                          v <- (1 - lambda) v + lambda v_other, and may be kept (unmixed or mixed, as cached) for such
//                          a layer to read
//   tq_bias_attention      every (token, head) on its own, its visible keys cut into n_splits ranges (decode steps,
//                          short runs; any sizes, both dtypes) + the merge of the ranges
//   tq_bias_attention_runs runs of new tokens (prompts): a block's queries share tiles of keys and values through
//                          shared memory
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define BA_MAX_DIM 256
#define BA_WARPS 4
#define BA_EPL (BA_MAX_DIM / 32)      // elements of a key or a value per lane

// ---------------------------------------------------------------------------------------
// One block per token walks the elements of its fused row.
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void bias_kv_write_kernel(const float* __restrict__ qkv, TA* __restrict__ q_out, TA* __restrict__ cache,
                                     float* __restrict__ v_keep, const float* __restrict__ v_other, float lambda,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                     const int* __restrict__ page_table, int table_stride, int page_size,
                                     int nh, int nkv, int dk, int dv, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const int nq = nh * dk, nk = nkv * dk, nv = nkv * dv;
    const float* row = qkv + (size_t)t * (nq + nk + nv);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q_out[(size_t)t * nq + i] = tq_from_float<TA>(row[i]);
    if (cache == nullptr && v_keep == nullptr) return;
    const int pos = positions[t];
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;
    const int page = TQ_CHECKED(table[TQ_CHECKED(pos / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
    const int slot = pos % page_size, dr = dk + dv;
    for (int i = threadIdx.x; i < nk + nv; i += blockDim.x) {
        float v = row[nq + i];
        int g, e;
        if (i < nk) { g = i / dk; e = i % dk; }
        else {
            const int j = i - nk;
            g = j / dv; e = dk + j % dv;
            if (v_other) v = (1.0f - lambda) * v + lambda * v_other[(size_t)t * nv + j];
            if (v_keep) v_keep[(size_t)t * nv + j] = v;
        }
        if (cache) cache[(((size_t)page * nkv + g) * page_size + slot) * dr + e] = tq_from_float<TA>(v);
    }
}

TQ_EXPORT int tq_bias_kv_write(const float* qkv, void* q_out, void* cache, int act_dtype, float* v_keep,
                               const float* v_other, float lambda, const int* positions, const int* seq_of_token,
                               const int* page_table, int table_stride, int page_size, int T_, int nh, int nkv, int dk,
                               int dv, int n_seqs, int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(nh >= 1 && nkv >= 1 && dk >= 1 && dv >= 1, "bias_kv_write: bad sizes %d %d %d %d", nh, nkv, dk, dv);
    const int n = nh * dk + nkv * (dk + dv);
    const int threads = n >= 1024 ? 512 : (n >= 256 ? 256 : 128);
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch(T_, threads, 0, stream)(bias_kv_write_kernel<TA>, qkv, (TA*)q_out, (TA*)cache, v_keep, v_other, lambda,
            positions, seq_of_token, page_table, table_stride, page_size, nh, nkv, dk, dv, n_seqs, n_pages)));
    TQ_CHECK_LAUNCH("bias_kv_write");
    return 0;
}

// ---------------------------------------------------------------------------------------
// The same split with norms and rotations on the way.  Per query and key head, in this order: an RMS norm with a weight
// shared by the heads (q_norm_w / k_norm_w fp32 [dk], x / sqrt(mean(x^2) + norm_eps) * w; null: none), the rotation
// by the token's position (the first rot_dims elements of each head, pairs of neighbours or of halves, angle =
// position * freq[i] in fp32, cos and sin multiplied by `mag`), then a unit norm (unit_eps > 0:
// x / sqrt(mean(x^2) + unit_eps); 0: left as it is).  Values: kv head g caches value head g / v_share of the row
// (v_share > 1: neighbouring key heads keep the same values), turned by position * v_freq[m] over all dv elements
// in the same pairing (v_freq fp32 [dv / 2]; null: as they are).
// Grid (token, groups of four query and key heads): a warp per head; the blocks of a token share out the copy of the values.
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128)
bias_kv_write_rot_kernel(const float* __restrict__ qkv, int row_stride, TA* __restrict__ q_out, TA* __restrict__ cache,
                         const float* __restrict__ freq, int rot_dims, int halves, float mag, float unit_eps,
                         const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float norm_eps,
                         const float* __restrict__ v_freq, int v_share,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                         const int* __restrict__ page_table, int table_stride, int page_size,
                         int nh, int nkv, int dk, int dv, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_head[4][BA_MAX_DIM];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nq = nh * dk, nk = nkv * dk, nv = nkv * dv, dr = dk + dv;
    const float* row = qkv + (size_t)t * row_stride;
    const int pos = positions[t];
    int page = 0;                      // without a cache (a layer that only reads another's) no table is looked at
    if (cache != nullptr) {
        const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;
        page = TQ_CHECKED(table[TQ_CHECKED(pos / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
    }
    const int slot = pos % page_size;
    if (cache != nullptr)
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < nv; i += gridDim.y * blockDim.x) {
            const int g = i / dv, e = i % dv;
            const float* vh = row + nq + nk + (size_t)(g / v_share) * dv;
            const float v = v_freq ? tq_rotated(vh, e, dv & ~1, halves, v_freq, pos) : vh[e];
            cache[(((size_t)page * nkv + g) * page_size + slot) * dr + dk + e] = tq_from_float<TA>(v);
        }
    const int head = blockIdx.y * 4 + warp;
    if (head >= nh + nkv || (head >= nh && cache == nullptr)) return;      // without a cache the rows may hold queries only
    const float* src = row + (size_t)head * dk;                // keys follow the queries in the row
    float* sh = s_head[warp];
    const float* nw = head < nh ? q_norm_w : k_norm_w;
    if (nw != nullptr) {
        float ss = 0.f;
        for (int e = lane; e < dk; e += 32) { const float x = src[e]; ss += x * x; }
        const float rs = 1.0f / sqrtf(tq_warp_sum(ss) / (float)dk + norm_eps);
        for (int e = lane; e < dk; e += 32) sh[e] = src[e] * rs * nw[e];
    } else {
        for (int e = lane; e < dk; e += 32) sh[e] = src[e];
    }
    __syncwarp();
    float v[BA_EPL];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < BA_EPL; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < dk ? tq_rotated(sh, e, rot_dims, halves, freq, pos) * (e < rot_dims ? mag : 1.0f) : 0.f;
        ss += v[j] * v[j];
    }
    float rs = 1.f;
    if (unit_eps > 0.f) rs = 1.0f / sqrtf(tq_warp_sum(ss) / (float)dk + unit_eps);
    TA* dst = head < nh ? q_out + ((size_t)t * nh + head) * dk
                        : (cache ? cache + (((size_t)page * nkv + (head - nh)) * page_size + slot) * dr : nullptr);
    if (dst == nullptr) return;
#pragma unroll
    for (int j = 0; j < BA_EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < dk) dst[e] = tq_from_float<TA>(v[j] * rs);
    }
}

// qkv: fp32 rows of row_stride floats that begin with [q | k | v] (v: nkv / v_share heads); freq: fp32 [rot_dims / 2]
// (null with rot_dims 0).
TQ_EXPORT int tq_bias_kv_write_rot(const float* qkv, int row_stride, void* q_out, void* cache, int act_dtype,
                                   const float* freq, int rot_dims, int halves, float mag, float unit_eps,
                                   const float* q_norm_w, const float* k_norm_w, float norm_eps, const float* v_freq,
                                   int v_share, const int* positions,
                                   const int* seq_of_token, const int* page_table, int table_stride, int page_size,
                                   int T_, int nh, int nkv, int dk, int dv, int n_seqs, int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(nh >= 1 && nkv >= 1 && dk >= 1 && dv >= 1 && dk <= BA_MAX_DIM, "bias_kv_write_rot: bad sizes %d %d %d %d", nh, nkv, dk, dv);
    TQ_REQUIRE(v_share >= 1 && nkv % v_share == 0, "bias_kv_write_rot: %d key heads cannot share values in groups of %d", nkv, v_share);
    TQ_REQUIRE(row_stride >= nh * dk + (cache ? nkv * dk + nkv / v_share * dv : 0), "bias_kv_write_rot: rows of %d floats do not hold the heads", row_stride);
    TQ_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk && (rot_dims == 0 || freq != nullptr),
               "bias_kv_write_rot: %d rotated elements of a head of %d", rot_dims, dk);
    TQ_REQUIRE(v_freq == nullptr || dv % 2 == 0, "bias_kv_write_rot: values of %d elements cannot be rotated in pairs", dv);
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch(dim3(T_, (nh + nkv + 3) / 4), 128, 0, stream)(bias_kv_write_rot_kernel<TA>, qkv, row_stride, (TA*)q_out, (TA*)cache, freq, rot_dims,
            halves, mag, unit_eps, q_norm_w, k_norm_w, norm_eps, v_freq, v_share, positions, seq_of_token, page_table, table_stride, page_size,
            nh, nkv, dk, dv, n_seqs, n_pages)));
    TQ_CHECK_LAUNCH("bias_kv_write_rot");
    return 0;
}

// ---------------------------------------------------------------------------------------
// What follows the weighted sums of two designs' attention, per (token, head), in fp32:
//   tq_heads_unrotate_gate   a head's output turned back by its own position (pair m by -position * v_freq[m] over all
//                            dv elements; null: not turned), times sigmoid of the head's gate logit (one per head, from
//                            a projection's fp32 rows)
//   tq_diff_combine          two maps' outputs a1, a2 of a head over the same values: o = a1 - lambda * a2,
//                            o / sqrt(mean(o^2) + eps) * out_scale, times sigmoid of the element's gate logit.  The
//                            maps lie as the attention kernels leave them with the maps of a key/value head's queries
//                            side by side: head (g, map, j) at g * 2 * per + map * per + j, per = heads / kv heads.
// A warp per (token, head), four a block.
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128)
heads_unrotate_gate_kernel(const TA* __restrict__ o, const float* __restrict__ gates, int gate_stride, int gate_off,
                           const float* __restrict__ v_freq, int halves, const int* __restrict__ positions,
                           TA* __restrict__ out, int T_, int nh, int dv) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_head[4][BA_MAX_DIM];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t item = (size_t)blockIdx.x * 4 + warp;
    if (item >= (size_t)T_ * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    float* sh = s_head[warp];
    const TA* src = o + item * dv;
    for (int e = lane; e < dv; e += 32) sh[e] = tq_to_float(src[e]);
    __syncwarp();
    const float z = gates[(size_t)t * gate_stride + gate_off + h];
    const float gate = 1.0f / (1.0f + expf(-z));
    const int pos = positions[t];
    for (int e = lane; e < dv; e += 32) {
        const float v = v_freq ? tq_rotated(sh, e, dv & ~1, halves, v_freq, -pos) : sh[e];
        out[item * dv + e] = tq_from_float<TA>(v * gate);
    }
}

TQ_EXPORT int tq_heads_unrotate_gate(const void* o, int act_dtype, const float* gates, int gate_stride, int gate_off,
                                     const float* v_freq, int halves, const int* positions, void* out, int T_, int nh, int dv,
                                     cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(nh >= 1 && dv >= 1 && dv <= BA_MAX_DIM, "heads_unrotate_gate: %d heads of %d values", nh, dv);
    TQ_REQUIRE(gate_off >= 0 && gate_off + nh <= gate_stride, "heads_unrotate_gate: the gates lie outside their rows");
    TQ_REQUIRE(v_freq == nullptr || dv % 2 == 0, "heads_unrotate_gate: values of %d elements cannot be rotated in pairs", dv);
    const long long items = (long long)T_ * nh;
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch((unsigned)((items + 3) / 4), 128, 0, stream)(heads_unrotate_gate_kernel<TA>, (const TA*)o, gates, gate_stride, gate_off,
            v_freq, halves, positions, (TA*)out, T_, nh, dv)));
    TQ_CHECK_LAUNCH("heads_unrotate_gate");
    return 0;
}

template <typename TA>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const TA* __restrict__ o, const float* __restrict__ gates, int gate_stride, int gate_off, float lambda,
                    float eps, float out_scale, TA* __restrict__ out, int T_, int nh, int nkv, int dv) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t item = (size_t)blockIdx.x * 4 + warp;
    if (item >= (size_t)T_ * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    const int per = nh / nkv, g = h / per, j = h % per;
    const TA* a1 = o + ((size_t)t * 2 * nh + (size_t)g * 2 * per + j) * dv;
    const TA* a2 = a1 + (size_t)per * dv;
    float v[BA_EPL];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < BA_EPL; ++k) {
        const int e = lane + 32 * k;
        v[k] = e < dv ? tq_to_float(a1[e]) - lambda * tq_to_float(a2[e]) : 0.f;
        ss += v[k] * v[k];
    }
    const float rs = out_scale / sqrtf(tq_warp_sum(ss) / (float)dv + eps);
    const float* gr = gates + (size_t)t * gate_stride + gate_off + (size_t)h * dv;
#pragma unroll
    for (int k = 0; k < BA_EPL; ++k) {
        const int e = lane + 32 * k;
        if (e < dv) out[item * dv + e] = tq_from_float<TA>(v[k] * rs / (1.0f + expf(-gr[e])));
    }
}

TQ_EXPORT int tq_diff_combine(const void* o, int act_dtype, const float* gates, int gate_stride, int gate_off, float lambda,
                              float eps, float out_scale, void* out, int T_, int nh, int nkv, int dv, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(nh >= 1 && nkv >= 1 && nh % nkv == 0 && dv >= 1 && dv <= BA_MAX_DIM, "diff_combine: %d heads on %d of %d values", nh, nkv, dv);
    TQ_REQUIRE(gate_off >= 0 && gate_off + nh * dv <= gate_stride, "diff_combine: the gates lie outside their rows");
    const long long items = (long long)T_ * nh;
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch((unsigned)((items + 3) / 4), 128, 0, stream)(diff_combine_kernel<TA>, (const TA*)o, gates, gate_stride, gate_off, lambda,
            eps, out_scale, (TA*)out, T_, nh, nkv, dv)));
    TQ_CHECK_LAUNCH("diff_combine");
    return 0;
}

// The visible positions of a query at `pos`, in order: [0, n_first) and [start, pos].
struct BaSpan {
    int n_first, start, count;
    __device__ __forceinline__ int at(int n) const { return n < n_first ? n : start + (n - n_first); }
};
// With cells (cell > 0) a query sees the positions of its own cell only: those from pos - pos % cell on, which is a
// window of pos % cell + 1 positions.
__device__ __forceinline__ int ba_window_at(int pos, int window, int cell) { return cell > 0 ? pos % cell + 1 : window; }
__device__ __forceinline__ BaSpan ba_span(int pos, int window, int keep_first) {
    BaSpan s;
    s.start = window > 0 ? max(0, pos + 1 - window) : 0;
    s.n_first = min(keep_first, s.start);
    s.count = s.n_first + (pos + 1 - s.start);
    return s;
}

// ---------------------------------------------------------------------------------------
// Token form: grid (T, heads, n_splits), 4 warps.  The block's range of the visible positions is walked key by key,
// warp w taking every fourth; a lane holds elements lane, lane + 32, ... of the key and of the value; online softmax
// per warp, merged through shared memory in warp order.  The sink enters as the first warp's starting state in the
// first range.  With n_splits > 1 the block's state (max, sum, weighted values) goes to `partial`.
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(BA_WARPS * 32)
bias_attention_kernel(const TA* __restrict__ q, const TA* __restrict__ cache, const float* __restrict__ bias, int far,
                      const float* __restrict__ sink, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int table_stride,
                      int page_size, int window, int keep_first, int cell, float scale, float softcap, TA* __restrict__ out,
                      float* __restrict__ partial, int n_splits, int nh, int nkv, int dk, int dv, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_m[BA_WARPS], s_l[BA_WARPS];
    __shared__ float s_acc[BA_WARPS][BA_MAX_DIM];
    const int t = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = h / (nh / nkv), dr = dk + dv;
    const int pos = positions[t];
    const BaSpan span = ba_span(pos, ba_window_at(pos, window, cell), cell > 0 ? 0 : keep_first);
    const int per = (span.count + n_splits - 1) / n_splits;
    const int n0 = split * per, n1 = min(span.count, n0 + per);
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;

    float qv[BA_EPL], acc[BA_EPL];
    const TA* qp = q + ((size_t)t * nh + h) * dk;
#pragma unroll
    for (int j = 0; j < BA_EPL; ++j) {
        const int e = lane + 32 * j;
        qv[j] = e < dk ? tq_to_float(qp[e]) * scale : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    if (sink != nullptr && split == 0 && warp == 0) { m = sink[h]; l = 1.f; }
    for (int n = n0 + warp; n < n1; n += BA_WARPS) {
        const int p = span.at(n);
        const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const TA* kp = cache + (((size_t)page * nkv + g) * page_size + p % page_size) * dr;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < BA_EPL; ++j) {
            const int e = lane + 32 * j;
            if (e < dk) s += qv[j] * tq_to_float(kp[e]);
        }
        s = tq_warp_sum(s);
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        if (bias) s += bias[(size_t)min(pos - p, far) * nh + h];
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);          // exp(-inf) = 0 on the first key
        const float pexp = expf(s - m_new);
        l = l * corr + pexp;
#pragma unroll
        for (int j = 0; j < BA_EPL; ++j) {
            const int e = lane + 32 * j;
            if (e < dv) acc[j] = acc[j] * corr + pexp * tq_to_float(kp[dk + e]);
        }
        m = m_new;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < BA_EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < dv) s_acc[warp][e] = acc[j];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < BA_WARPS; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f;
    float f[BA_WARPS];
#pragma unroll
    for (int w = 0; w < BA_WARPS; ++w) {
        f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);
        L += s_l[w] * f[w];
    }
    if (n_splits > 1) {
        float* pr = partial + (((size_t)t * nh + h) * n_splits + split) * (dv + 2);
        if (threadIdx.x == 0) { pr[0] = M; pr[1] = L; }
        for (int e = threadIdx.x; e < dv; e += blockDim.x) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < BA_WARPS; ++w) v += s_acc[w][e] * f[w];
            pr[2 + e] = v;
        }
        return;
    }
    TA* op = out + ((size_t)t * nh + h) * dv;
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < BA_WARPS; ++w) v += s_acc[w][e] * f[w];
        op[e] = tq_from_float<TA>(v / L);
    }
}

// The ranges of one (token, head), added up in range order: grid (T * heads).
template <typename TA>
__global__ void bias_attention_merge_kernel(const float* __restrict__ partial, int n_splits, int dv, TA* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const float* p = partial + (size_t)blockIdx.x * n_splits * (dv + 2);
    float M = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) M = fmaxf(M, p[(size_t)sp * (dv + 2)]);
    float L = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
        const float ms = p[(size_t)sp * (dv + 2)];
        if (ms != -INFINITY) L += p[(size_t)sp * (dv + 2) + 1] * expf(ms - M);
    }
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float a = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float ms = p[(size_t)sp * (dv + 2)];
            if (ms != -INFINITY) a += p[(size_t)sp * (dv + 2) + 2 + e] * expf(ms - M);
        }
        out[(size_t)blockIdx.x * dv + e] = tq_from_float<TA>(a / L);
    }
}

TQ_EXPORT int tq_bias_attention(const void* q, const void* cache, int act_dtype, const float* bias, int far,
                                const float* sink, const int* positions, const int* seq_of_token,
                                const int* page_table, int table_stride, int page_size, int window, int keep_first, int cell,
                                float scale, float softcap, void* out, float* partial, int n_splits, int T_, int nh, int nkv, int dk,
                                int dv, int n_seqs, int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(dk >= 1 && dk <= BA_MAX_DIM && dv >= 1 && dv <= BA_MAX_DIM, "bias_attention: key size %d or value size %d exceeds %d", dk, dv, BA_MAX_DIM);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "bias_attention: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE(nh <= 65535 && n_splits >= 1 && n_splits <= 65535, "bias_attention: %d heads or %d ranges exceed the grid limit", nh, n_splits);
    TQ_REQUIRE(window >= 0 && keep_first >= 0 && far >= 0, "bias_attention: negative window, kept positions or distance");
    TQ_REQUIRE(n_splits == 1 || partial != nullptr, "bias_attention: %d ranges need scratch for their states", n_splits);
    dim3 grid(T_, nh, n_splits);
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch(grid, BA_WARPS * 32, 0, stream)(bias_attention_kernel<TA>, (const TA*)q, (const TA*)cache, bias, far, sink,
            positions, seq_of_token, page_table, table_stride, page_size, window, keep_first, cell, scale, softcap, (TA*)out, partial,
            n_splits, nh, nkv, dk, dv, n_seqs, n_pages)));
    TQ_CHECK_LAUNCH("bias_attention");
    if (n_splits > 1) {
        TQ_DISPATCH(act_dtype, TA,
            (tq_launch(T_ * nh, dv >= 128 ? 128 : 64, 0, stream)(bias_attention_merge_kernel<TA>, partial, n_splits, dv, (TA*)out)));
        TQ_CHECK_LAUNCH("bias_attention_merge");
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// Token form for grouped queries, bfloat16, key and value sizes of 32, 64 or 128: grid (token x head chunks, kv head,
// range), 4 warps.  A block keeps up to GC query heads of one key/value head in registers and reads every cached row
// once for all of them: a row's key is read by LPK = DK / 8 lanes with one 16-byte load each, so a warp covers
// 32 / LPK rows per instruction and eight rows per iteration; the value's 16-byte pieces are shared out over the same
// lanes.  The loads are cp.async copies into a ring in shared memory, two iterations ahead of the one being computed,
// every lane copying and reading back only its own 16 bytes (no barrier between the lanes or warps).  Online softmax per head and
// lane group (fp32), merged over the lane groups by shuffles and over the warps through shared memory, in a fixed
// order.  The ranges' states go to `partial` as in the form above and are joined by the same merge.
// bias_t: [heads][far + 1].
// ---------------------------------------------------------------------------------------
#define BG_STAGES 3
__device__ __forceinline__ void br_copy16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
struct BaRaw { uint4 v; };
__device__ __forceinline__ BaRaw ba_fetch(const __nv_bfloat16* p) { BaRaw r; r.v = *reinterpret_cast<const uint4*>(p); return r; }
__device__ __forceinline__ void ba_widen(const BaRaw& r, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

template <int DK, int DV, int GC>
__global__ void __launch_bounds__(BA_WARPS * 32)
bias_attention_group_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                            const float* __restrict__ bias_t, int far, const float* __restrict__ sink,
                            const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ page_table, int table_stride, int page_size, int window,
                            int keep_first, int cell, float scale, float softcap, __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                            int n_splits, int nh, int nkv, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    constexpr int LPK = DK / 8, KPI = 32 / LPK, LOADS = KPI >= 8 ? 1 : 8 / KPI, GS = KPI * LOADS;
    constexpr int NV8 = DV / 8, NVC = NV8 > LPK ? NV8 / LPK : 1, DR = DK + DV;
    __shared__ float s_m[BA_WARPS][GC], s_l[BA_WARPS][GC];
    __shared__ float s_acc[BA_WARPS][GC][DV];
    const int G_all = nh / nkv;
    const int chunks = (G_all + GC - 1) / GC;
    const int t = blockIdx.x / chunks, chunk = blockIdx.x - t * chunks, g = blockIdx.y, split = blockIdx.z;
    const int h0 = g * G_all + chunk * GC;                   // the block's first head
    const int G = min(GC, G_all - chunk * GC);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPK, part = lane / LPK;           // part: which of the KPI rows of a load
    const int pos = positions[t];
    const BaSpan span = ba_span(pos, ba_window_at(pos, window, cell), cell > 0 ? 0 : keep_first);
    int per = (span.count + n_splits - 1) / n_splits;
    per = (per + GS - 1) / GS * GS;
    const int n0 = split * per, n1 = min(span.count, n0 + per);
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;

    // the ring: [warp][stage][a key and NVC value pieces per load][lane] of 16 bytes, a lane's own slots only
    constexpr int SLOTS = LOADS * (1 + NVC);
    extern __shared__ __align__(16) uint4 ba_ring[];
    uint4* ring = ba_ring + (size_t)warp * BG_STAGES * SLOTS * 32 + lane;
    auto copy_group = [&](int base, int stage) {
        uint4* dst = ring + (size_t)stage * SLOTS * 32;
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            const int n = min(base + j * KPI + part, n1 - 1);            // rows past the range repeat its last row (masked below)
            const int p = span.at(n);
            const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
            const __nv_bfloat16* row = cache + (((size_t)page * nkv + g) * page_size + p % page_size) * DR;
            br_copy16(dst + (j * (1 + NVC)) * 32, row + sub * 8);
#pragma unroll
            for (int c = 0; c < NVC; ++c)
                if (sub + c * LPK < NV8) br_copy16(dst + (j * (1 + NVC) + 1 + c) * 32, row + DK + (sub + c * LPK) * 8);
        }
    };
    int next_base = n0 + warp * GS, next_stage = 0, stage = 0;
#pragma unroll
    for (int i = 0; i < BG_STAGES - 1; ++i) {                 // one commit per group, also past the end: the count is uniform
        if (next_base < n1) copy_group(next_base, next_stage);
        asm volatile("cp.async.commit_group;" ::: "memory");
        next_base += BA_WARPS * GS;
        next_stage = next_stage + 1 == BG_STAGES ? 0 : next_stage + 1;
    }

    float qv[GC][8], acc[GC][NVC][8], m[GC], l[GC];
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
        if (sink != nullptr && split == 0 && warp == 0 && part == 0 && h < G) { m[h] = sink[h0 + h]; l[h] = 1.f; }
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (h < G) { const BaRaw r = ba_fetch(q + ((size_t)t * nh + h0 + h) * DK + sub * 8); ba_widen(r, f); }
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[h][i] = f[i] * scale;
#pragma unroll
        for (int c = 0; c < NVC; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[h][c][i] = 0.f;
    }
    for (int base = n0 + warp * GS; base < n1; base += BA_WARPS * GS) {
        // the slot filled now was read one iteration ago, and what was read there has been used since
        if (next_base < n1) copy_group(next_base, next_stage);
        asm volatile("cp.async.commit_group;" ::: "memory");
        next_base += BA_WARPS * GS;
        next_stage = next_stage + 1 == BG_STAGES ? 0 : next_stage + 1;
        asm volatile("cp.async.wait_group %0;" ::"n"(BG_STAGES - 1) : "memory");   // all but the newest groups have landed: this one has
        const uint4* src = ring + (size_t)stage * SLOTS * 32;
        stage = stage + 1 == BG_STAGES ? 0 : stage + 1;
        float kf[LOADS][8], vf[LOADS][NVC][8];
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            BaRaw r;
            r.v = src[(j * (1 + NVC)) * 32];
            ba_widen(r, kf[j]);
#pragma unroll
            for (int c = 0; c < NVC; ++c) {
                if (sub + c * LPK < NV8) { r.v = src[(j * (1 + NVC) + 1 + c) * 32]; ba_widen(r, vf[j][c]); }
                else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) vf[j][c][i] = 0.f;
                }
            }
        }
        float s[LOADS][GC];
#pragma unroll
        for (int j = 0; j < LOADS; ++j)
#pragma unroll
            for (int h = 0; h < GC; ++h) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) d = fmaf(qv[h][i], kf[j][i], d);
                s[j][h] = d;
            }
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < LOADS; ++j)
#pragma unroll
                for (int h = 0; h < GC; ++h) s[j][h] += __shfl_xor_sync(0xffffffffu, s[j][h], o);
#pragma unroll
        for (int h = 0; h < GC; ++h) {
            if (h >= G) continue;
            float mx = m[h];
#pragma unroll
            for (int j = 0; j < LOADS; ++j) {
                const int n = base + j * KPI + part;
                if (n < n1) {
                    if (softcap > 0.f) s[j][h] = softcap * tanhf(s[j][h] / softcap);
                    if (bias_t) s[j][h] += __ldg(bias_t + (size_t)(h0 + h) * (far + 1) + min(pos - span.at(n), far));
                } else s[j][h] = -INFINITY;
                mx = fmaxf(mx, s[j][h]);
            }
            if (mx == -INFINITY) continue;                 // nothing visible yet for this lane group
            const float corr = expf(m[h] - mx);
            float lsum = l[h] * corr;
#pragma unroll
            for (int c = 0; c < NVC; ++c)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[h][c][i] *= corr;
#pragma unroll
            for (int j = 0; j < LOADS; ++j) {
                const float pe = expf(s[j][h] - mx);       // exp(-inf) = 0 for masked rows
                lsum += pe;
#pragma unroll
                for (int c = 0; c < NVC; ++c)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[h][c][i] = fmaf(pe, vf[j][c][i], acc[h][c][i]);
            }
            m[h] = mx; l[h] = lsum;
        }
    }
    // the warp's KPI lane groups, joined by shuffles (the same order for every launch)
#pragma unroll
    for (int h = 0; h < GC; ++h) {
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[h], o);
            const float lo = __shfl_xor_sync(0xffffffffu, l[h], o);
            const float M = fmaxf(m[h], mo);
            const float fa = m[h] == -INFINITY ? 0.f : expf(m[h] - M), fb = mo == -INFINITY ? 0.f : expf(mo - M);
            l[h] = l[h] * fa + lo * fb;
#pragma unroll
            for (int c = 0; c < NVC; ++c)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float ao = __shfl_xor_sync(0xffffffffu, acc[h][c][i], o);
                    acc[h][c][i] = acc[h][c][i] * fa + ao * fb;
                }
            m[h] = M;
        }
        if (lane == 0) { s_m[warp][h] = m[h]; s_l[warp][h] = l[h]; }
        if (part == 0) {
#pragma unroll
            for (int c = 0; c < NVC; ++c)
                if (sub + c * LPK < NV8) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) s_acc[warp][h][(sub + c * LPK) * 8 + i] = acc[h][c][i];
                }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * DV; idx += blockDim.x) {
        const int h = idx / DV, d = idx % DV;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < BA_WARPS; ++w) M = fmaxf(M, s_m[w][h]);
        float L = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < BA_WARPS; ++w) {
            const float f = s_m[w][h] == -INFINITY ? 0.f : expf(s_m[w][h] - M);
            L += s_l[w][h] * f;
            a += s_acc[w][h][d] * f;
        }
        if (n_splits == 1) {
            out[((size_t)t * nh + h0 + h) * DV + d] = __float2bfloat16_rn(a / L);
            continue;
        }
        float* dst = partial + (((size_t)t * nh + h0 + h) * n_splits + split) * (DV + 2);
        dst[2 + d] = a;
        if (d == 0) { dst[0] = M; dst[1] = L; }
    }
}

// Heads a block of the grouped form keeps for `per_kv` query heads per key/value head and this shape (0: the shape
// is not built).
static int ba_group_heads(int dk, int dv, int per_kv) {
    if (!((dk == 32 || dk == 64 || dk == 128) && (dv == 32 || dv == 64 || dv == 128))) return 0;
    const int nvc = dv / 8 > dk / 8 ? dv / dk : 1;
    int gc = per_kv >= 8 ? 8 : (per_kv > 2 ? 4 : per_kv);
    if (dk == 128 && gc > 4) gc = 4;          // four loads of a lane in flight: eight heads would spill registers
    while (gc * nvc > 8 && gc > 1) gc >>= 1;
    return gc;
}
TQ_EXPORT int tq_bias_attention_group_heads(int dk, int dv, int per_kv) { return ba_group_heads(dk, dv, per_kv); }

TQ_EXPORT int tq_bias_attention_group(const void* q, const void* cache, const float* bias_t, int far, const float* sink,
                                      const int* positions, const int* seq_of_token, const int* page_table,
                                      int table_stride, int page_size, int window, int keep_first, int cell, float scale, float softcap, void* out,
                                      float* partial, int n_splits, int T_, int nh, int nkv, int dk, int dv, int n_seqs,
                                      int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "bias_attention_group: %d heads are not a multiple of %d key/value heads", nh, nkv);
    const int gc = ba_group_heads(dk, dv, nh / nkv);
    TQ_REQUIRE(gc > 0, "bias_attention_group: key size %d and value size %d must each be 32, 64 or 128", dk, dv);
    TQ_REQUIRE(window >= 0 && keep_first >= 0 && far >= 0, "bias_attention_group: negative window, kept positions or distance");
    TQ_REQUIRE(n_splits >= 1 && n_splits <= 65535 && nkv <= 65535, "bias_attention_group: %d ranges or %d key/value heads exceed the grid limit", n_splits, nkv);
    TQ_REQUIRE(n_splits == 1 || partial != nullptr, "bias_attention_group: %d ranges need scratch for their states", n_splits);
    const int chunks = (nh / nkv + gc - 1) / gc;
    dim3 grid(T_ * chunks, nkv, n_splits);
    bool done = false;
#define BG_CASE(DK_, DV_, GC_)                                                                                        \
    if (!done && dk == DK_ && dv == DV_ && gc == GC_) {                                                               \
        constexpr int kpi = 32 / (DK_ / 8), loads = kpi >= 8 ? 1 : 8 / kpi, nvc = DV_ / 8 > DK_ / 8 ? DV_ / DK_ : 1;   \
        constexpr int ring_bytes = BA_WARPS * BG_STAGES * loads * (1 + nvc) * 32 * 16;                                \
        static bool configured = false;                                                                               \
        if (!configured) {                                                                                            \
            cudaError_t e = cudaFuncSetAttribute(bias_attention_group_kernel<DK_, DV_, GC_>,                           \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes);            \
            if (e != cudaSuccess) TQ_FAIL(-1, "bias_attention_group: %d bytes of shared memory refused: %s", ring_bytes, cudaGetErrorString(e)); \
            configured = true;                                                                                        \
        }                                                                                                             \
        tq_launch(grid, BA_WARPS * 32, ring_bytes, stream)(bias_attention_group_kernel<DK_, DV_, GC_>, (const __nv_bfloat16*)q,  \
            (const __nv_bfloat16*)cache, bias_t, far, sink, positions, seq_of_token, page_table, table_stride, page_size, \
            window, keep_first, cell, scale, softcap, (__nv_bfloat16*)out, partial, n_splits, nh, nkv, n_seqs, n_pages);             \
        done = true;                                                                                                  \
    }
#define BG_SHAPE(DK_, DV_) BG_CASE(DK_, DV_, 1) BG_CASE(DK_, DV_, 2) BG_CASE(DK_, DV_, 4)
    BG_SHAPE(32, 32) BG_SHAPE(64, 32) BG_SHAPE(64, 64) BG_SHAPE(128, 32) BG_SHAPE(128, 64) BG_SHAPE(128, 128)
    BG_CASE(32, 32, 8) BG_CASE(64, 32, 8) BG_CASE(64, 64, 8)
    BG_CASE(32, 64, 1) BG_CASE(32, 64, 2) BG_CASE(32, 64, 4) BG_CASE(64, 128, 1) BG_CASE(64, 128, 2) BG_CASE(64, 128, 4)
    BG_CASE(32, 128, 1) BG_CASE(32, 128, 2)
#undef BG_SHAPE
#undef BG_CASE
    TQ_REQUIRE(done, "bias_attention_group: no kernel for sizes %d, %d with %d heads a block", dk, dv, gc);
    TQ_CHECK_LAUNCH("bias_attention_group");
    if (n_splits > 1) {
        tq_launch(T_ * nh, dv >= 128 ? 128 : 64, 0, stream)(bias_attention_merge_kernel<__nv_bfloat16>, partial, n_splits, dv, (__nv_bfloat16*)out);
        TQ_CHECK_LAUNCH("bias_attention_merge");
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// Runs of new tokens (prompts), bfloat16, on tensor cores (mma.sync m16n8k16, fp32 accumulation).  A block of four
// warps takes 64 consecutive queries of one (sequence, head), a warp 16 of them; the keys come a page at a time (64
// positions: one contiguous piece of the cache, key and value side by side) through a two-stage cp.async ring in
// shared memory.  Only pages that some query of the block can see are walked: the kept first pages, then the pages
// of the window; the mask inside a page is exact.  S = Q K^T lives in accumulator fragments, where the bias is
// added, the mask applied and the online softmax kept per row (fp32); the weights, rounded to bfloat16, are the
// left operand of the second product with the values read transposed from the same rows.  The sink joins the
// denominator at the end.  DK, DV: key and value size (multiples of 16 up to 128); the page size is 64.
// ---------------------------------------------------------------------------------------
#define BR_Q 64
#define BR_K 64
#define BR_WARPS 4

__device__ __forceinline__ void br_ldsm4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void br_ldsm4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void br_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t br_pack(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int DK, int DV>
__global__ void __launch_bounds__(BR_WARPS * 32, 3)
bias_attention_runs_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                           const float* __restrict__ bias_t, int far, const float* __restrict__ sink,
                           const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                           const int* __restrict__ page_table, int table_stride, int window, int keep_first, int cell,
                           float scale, float softcap, __nv_bfloat16* __restrict__ out, int nh, int nkv, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    constexpr int DR = DK + DV, LD = DR + 8;                 // a shared-memory row: key, value, 16 bytes of padding
    extern __shared__ __align__(16) uint8_t br_smem[];
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(br_smem);      // [2][BR_K][LD]
    // the bias of the distances a tile's keys can have from the block's queries, staged per tile: element x is the
    // bias at distance (pos0 - tile's first position - (BR_K - 1)) + x, clamped into the table
    __shared__ float s_bias[2][BR_Q + BR_K];
    // the grid is (head, sequence, block of queries from the last to the first): blocks start in that order, so the
    // blocks with the most pages to walk (late queries) run first and the short ones fill the GPU's last round, and
    // the heads that share a key/value head run side by side and meet in the L2
    const int seq = blockIdx.y, h = blockIdx.x;
    const int t0 = cu_seqlens[seq], n_run = cu_seqlens[seq + 1] - t0;
    const int a0 = (int)(gridDim.z - 1 - blockIdx.z) * BR_Q; // first query of the block within the run
    if (a0 >= n_run) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = h / (nh / nkv);
    const int pos0 = seq_start[seq] + a0;                    // position of the block's first query
    const int n_q = min(BR_Q, n_run - a0);
    const int pos_last = pos0 + n_q - 1;
    const int* table = page_table + (size_t)seq * table_stride;
    // pages to walk: [0, kept) and [first, last]
    // with cells, the block's first query sees back to the start of its cell, the later ones no further
    const int first = cell > 0 ? (pos0 - pos0 % cell) / BR_K : (window > 0 ? max(0, pos0 + 1 - window) / BR_K : 0);
    const int last = pos_last / BR_K;
    const int kept = window > 0 && cell == 0 ? min((keep_first + BR_K - 1) / BR_K, first) : 0;
    const int n_tiles = kept + (last - first + 1);

    auto load_tile = [&](int i, int stage) {
        const int pg = i < kept ? i : first + (i - kept);
        const int page = TQ_CHECKED(table[TQ_CHECKED(pg, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const __nv_bfloat16* src = cache + ((size_t)max(page, 0) * nkv + g) * BR_K * DR;
        __nv_bfloat16* dst = tiles + (size_t)stage * BR_K * LD;
        constexpr int CPR = DR / 8;                          // 16-byte pieces of a row
        for (int c = threadIdx.x; c < BR_K * CPR; c += BR_WARPS * 32) {
            const int r = c / CPR, k = c % CPR;
            br_copy16(dst + r * LD + k * 8, src + r * DR + k * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (bias_t != nullptr && threadIdx.x < BR_Q + BR_K - 1) {
            const int d = pos0 - pg * BR_K - (BR_K - 1) + (int)threadIdx.x;
            s_bias[stage][threadIdx.x] = __ldg(bias_t + (size_t)h * (far + 1) + min(max(d, 0), far));
        }
    };
    load_tile(0, 0);

    // this warp's 16 queries as left-operand fragments
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;           // the thread's two rows within the block
    uint32_t qf[DK / 16][4];
    {
        const __nv_bfloat16* q_lo = q + ((size_t)(t0 + a0 + r_lo) * nh + h) * DK + (lane & 3) * 2;
        const __nv_bfloat16* q_hi = q + ((size_t)(t0 + a0 + r_hi) * nh + h) * DK + (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            qf[ks][0] = r_lo < n_q ? *reinterpret_cast<const uint32_t*>(q_lo + ks * 16) : 0u;
            qf[ks][1] = r_hi < n_q ? *reinterpret_cast<const uint32_t*>(q_hi + ks * 16) : 0u;
            qf[ks][2] = r_lo < n_q ? *reinterpret_cast<const uint32_t*>(q_lo + ks * 16 + 8) : 0u;
            qf[ks][3] = r_hi < n_q ? *reinterpret_cast<const uint32_t*>(q_hi + ks * 16 + 8) : 0u;
        }
    }
    const bool biased = bias_t != nullptr;
    const float sink_h = sink ? sink[h] : -INFINITY;
    float m_lo = sink_h, m_hi = sink_h, l_lo = 0.f, l_hi = 0.f;
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    const int i_lo = pos0 + r_lo, i_hi = pos0 + r_hi;                    // the two rows' positions

    for (int it = 0; it < n_tiles; ++it) {
        const int stage = it & 1;
        if (it + 1 < n_tiles) {
            load_tile(it + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* tile = tiles + (size_t)stage * BR_K * LD;
        const int p_base = (it < kept ? it : first + (it - kept)) * BR_K;     // position of the tile's first key
        // a warp whose rows see nothing of this tile skips it (the tile lies wholly behind its last query)
        const bool any = p_base <= pos0 + min(warp * 16 + 15, n_q - 1);
        if (any) {
            float s[BR_K / 8][4];
#pragma unroll
            for (int n = 0; n < BR_K / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
                for (int n = 0; n < BR_K / 8; n += 2) {
                    uint32_t b[4];
                    const int mi = lane >> 3;
                    br_ldsm4(b, tile + ((n + (mi >> 1)) * 8 + (lane & 7)) * LD + ks * 16 + (mi & 1) * 8);
                    br_mma(s[n], qf[ks], b[0], b[1]);
                    br_mma(s[n + 1], qf[ks], b[2], b[3]);
                }
            }
            // scale, bias, mask; the rows' maxima
            const float* sb = s_bias[stage];
            const int d_min = pos0 - p_base - (BR_K - 1);
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int n = 0; n < BR_K / 8; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int p = p_base + n * 8 + (lane & 3) * 2 + (c & 1);
                    const int i = (c & 2) ? i_hi : i_lo;
                    const int d = i - p;
                    const bool see = d >= 0 && (cell > 0 ? p >= i - i % cell : (window == 0 || d < window || p < keep_first));
                    float v = s[n][c] * scale;
                    if (softcap > 0.f) v = softcap * tanhf(v / softcap);
                    if (biased) v += sb[min(max(d - d_min, 0), BR_Q + BR_K - 2)];
                    v = see ? v : -INFINITY;
                    s[n][c] = v;
                    if (c & 2) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
                }
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
            const float u_lo = mn_lo == -INFINITY ? 0.f : mn_lo, u_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
            const float c_lo = __expf(m_lo - u_lo), c_hi = __expf(m_hi - u_hi);  // exp(-inf) = 0 before the first key
            m_lo = mn_lo; m_hi = mn_hi;
            l_lo *= c_lo; l_hi *= c_hi;
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) { o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi; }
#pragma unroll
            for (int n = 0; n < BR_K / 8; ++n) {
                // the weights keep eight bits as the second product's operand: the fast exponential does
                s[n][0] = __expf(s[n][0] - u_lo); s[n][1] = __expf(s[n][1] - u_lo);
                s[n][2] = __expf(s[n][2] - u_hi); s[n][3] = __expf(s[n][3] - u_hi);
                l_lo += s[n][0] + s[n][1];
                l_hi += s[n][2] + s[n][3];
            }
            // O += P V: sixteen keys at a time
#pragma unroll
            for (int kk = 0; kk < BR_K / 16; ++kk) {
                uint32_t a[4];
                a[0] = br_pack(s[2 * kk][0], s[2 * kk][1]);
                a[1] = br_pack(s[2 * kk][2], s[2 * kk][3]);
                a[2] = br_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                a[3] = br_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int n = 0; n < DV / 8; n += 2) {
                    uint32_t b[4];
                    const int mi = lane >> 3;
                    br_ldsm4_t(b, tile + (kk * 16 + (mi & 1) * 8 + (lane & 7)) * LD + DK + (n + (mi >> 1)) * 8);
                    br_mma(o[n], a, b[0], b[1]);
                    br_mma(o[n + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();               // the stage is loaded again two tiles on
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (sink) { l_lo += expf(sink_h - m_lo); l_hi += expf(sink_h - m_hi); }
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
    __nv_bfloat16* o_lo = out + ((size_t)(t0 + a0 + r_lo) * nh + h) * DV + (lane & 3) * 2;
    __nv_bfloat16* o_hi = out + ((size_t)(t0 + a0 + r_hi) * nh + h) * DV + (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        if (r_lo < n_q) *reinterpret_cast<uint32_t*>(o_lo + n * 8) = br_pack(o[n][0] * inv_lo, o[n][1] * inv_lo);
        if (r_hi < n_q) *reinterpret_cast<uint32_t*>(o_hi + n * 8) = br_pack(o[n][2] * inv_hi, o[n][3] * inv_hi);
    }
}

// ---------------------------------------------------------------------------------------
// Token form on tensor cores, bfloat16, for several query heads per key/value head: the sixteen rows of
// mma.sync m16n8k16 are up to sixteen heads of one (token, key/value head).  Grid (token, key/value head x chunks of
// 16 heads, key range), four warps; the visible positions are walked in tiles of 16 absolute positions (a tile lies
// in one page: one contiguous piece of the cache), the kept first tiles and then the window's; warp w takes every
// fourth tile of the block's range through a two-stage cp.async ring of its own.  Scores, mask, bias and online
// softmax on the accumulator fragments as in the kernel for runs; the warps' states are joined through shared
// memory in warp order, the ranges' by bias_attention_merge.  The page size is a multiple of 16.
// ---------------------------------------------------------------------------------------
#define BH_K 16
template <int DK, int DV>
__global__ void __launch_bounds__(BA_WARPS * 32, 3)
bias_attention_heads_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                            const float* __restrict__ bias_t, int far, const float* __restrict__ sink,
                            const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ page_table, int table_stride, int page_size, int window,
                            int keep_first, int cell, float scale, float softcap, __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                            int n_splits, int nh, int nkv, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    constexpr int DR = DK + DV, LD = DR + 8;
    constexpr int STAGE = BH_K * LD;                         // elements of a warp's stage
    extern __shared__ __align__(16) uint8_t bh_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(bh_smem) + (size_t)warp * 2 * STAGE;
    const int G_all = nh / nkv;
    const int chunks = (G_all + 15) / 16;
    const int t = blockIdx.x, g = blockIdx.y / chunks, chunk = blockIdx.y - g * chunks, split = blockIdx.z;
    const int h0 = g * G_all + chunk * 16;
    const int G = min(16, G_all - chunk * 16);
    const int pos = positions[t];
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;
    if (cell > 0) { window = pos % cell + 1; keep_first = 0; }
    const int start = window > 0 ? max(0, pos + 1 - window) : 0;
    const int first = start / BH_K, last = pos / BH_K;
    const int kept = window > 0 ? min((keep_first + BH_K - 1) / BH_K, first) : 0;
    const int n_tiles = kept + (last - first + 1);
    const int per = (n_tiles + n_splits - 1) / n_splits;
    const int i0 = split * per, i1 = min(n_tiles, i0 + per);

    auto load_tile = [&](int i, int stage) {
        const int p0 = (i < kept ? i : first + (i - kept)) * BH_K;
        const int page = TQ_CHECKED(table[TQ_CHECKED(p0 / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const __nv_bfloat16* src = cache + (((size_t)max(page, 0) * nkv + g) * page_size + p0 % page_size) * DR;
        __nv_bfloat16* dst = ring + (size_t)stage * STAGE;
        constexpr int CPR = DR / 8;
        for (int c = lane; c < BH_K * CPR; c += 32) {
            const int r = c / CPR, k = c % CPR;
            br_copy16(dst + r * LD + k * 8, src + r * DR + k * 8);
        }
    };
    if (i0 + warp < i1) load_tile(i0 + warp, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    const int r_lo = lane >> 2, r_hi = r_lo + 8;             // the thread's two rows: heads h0 + r
    uint32_t qf[DK / 16][4];
    {
        const __nv_bfloat16* q_lo = q + ((size_t)t * nh + h0 + r_lo) * DK + (lane & 3) * 2;
        const __nv_bfloat16* q_hi = q + ((size_t)t * nh + h0 + r_hi) * DK + (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            qf[ks][0] = r_lo < G ? *reinterpret_cast<const uint32_t*>(q_lo + ks * 16) : 0u;
            qf[ks][1] = r_hi < G ? *reinterpret_cast<const uint32_t*>(q_hi + ks * 16) : 0u;
            qf[ks][2] = r_lo < G ? *reinterpret_cast<const uint32_t*>(q_lo + ks * 16 + 8) : 0u;
            qf[ks][3] = r_hi < G ? *reinterpret_cast<const uint32_t*>(q_hi + ks * 16 + 8) : 0u;
        }
    }
    const float* b_lo = bias_t && r_lo < G ? bias_t + (size_t)(h0 + r_lo) * (far + 1) : nullptr;
    const float* b_hi = bias_t && r_hi < G ? bias_t + (size_t)(h0 + r_hi) * (far + 1) : nullptr;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

    int stage = 0;
    for (int i = i0 + warp; i < i1; i += BA_WARPS) {
        if (i + BA_WARPS < i1) load_tile(i + BA_WARPS, stage ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncwarp();                                       // every lane's pieces of this tile have landed
        const __nv_bfloat16* tile = ring + (size_t)stage * STAGE;
        const int p_base = (i < kept ? i : first + (i - kept)) * BH_K;
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        const int mi = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            uint32_t b[4];
            br_ldsm4(b, tile + ((mi >> 1) * 8 + (lane & 7)) * LD + ks * 16 + (mi & 1) * 8);
            br_mma(s[0], qf[ks], b[0], b[1]);
            br_mma(s[1], qf[ks], b[2], b[3]);
        }
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int p = p_base + n * 8 + (lane & 3) * 2 + (c & 1);
                const int d = pos - p;
                const bool see = d >= 0 && (window == 0 || d < window || p < keep_first);
                const float* bh = (c & 2) ? b_hi : b_lo;
                float v = s[n][c] * scale;
                if (softcap > 0.f) v = softcap * tanhf(v / softcap);
                if (bh && see) v += __ldg(bh + min(d, far));
                v = see ? v : -INFINITY;
                s[n][c] = v;
                if (c & 2) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float u_lo = mn_lo == -INFINITY ? 0.f : mn_lo, u_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float c_lo = __expf(m_lo - u_lo), c_hi = __expf(m_hi - u_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        l_lo *= c_lo; l_hi *= c_hi;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) { o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi; }
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            s[n][0] = __expf(s[n][0] - u_lo); s[n][1] = __expf(s[n][1] - u_lo);
            s[n][2] = __expf(s[n][2] - u_hi); s[n][3] = __expf(s[n][3] - u_hi);
            l_lo += s[n][0] + s[n][1];
            l_hi += s[n][2] + s[n][3];
        }
        uint32_t a[4];
        a[0] = br_pack(s[0][0], s[0][1]);
        a[1] = br_pack(s[0][2], s[0][3]);
        a[2] = br_pack(s[1][0], s[1][1]);
        a[3] = br_pack(s[1][2], s[1][3]);
#pragma unroll
        for (int n = 0; n < DV / 8; n += 2) {
            uint32_t b[4];
            br_ldsm4_t(b, tile + ((mi & 1) * 8 + (lane & 7)) * LD + DK + (n + (mi >> 1)) * 8);
            br_mma(o[n], a, b[0], b[1]);
            br_mma(o[n + 1], a, b[2], b[3]);
        }
        __syncwarp();                                       // the stage is filled again two tiles on
        stage ^= 1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    // the warps' states meet in shared memory (the rings are done with): [warp][row] max and sum, [warp][row][DV]
    __syncthreads();
    float* s_m = reinterpret_cast<float*>(bh_smem);
    float* s_l = s_m + BA_WARPS * 16;
    float* s_o = s_l + BA_WARPS * 16;
    if ((lane & 3) == 0) {
        s_m[warp * 16 + r_lo] = m_lo; s_l[warp * 16 + r_lo] = l_lo;
        s_m[warp * 16 + r_hi] = m_hi; s_l[warp * 16 + r_hi] = l_hi;
    }
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        float* lo = s_o + ((size_t)warp * 16 + r_lo) * DV + n * 8 + (lane & 3) * 2;
        float* hi = s_o + ((size_t)warp * 16 + r_hi) * DV + n * 8 + (lane & 3) * 2;
        lo[0] = o[n][0]; lo[1] = o[n][1]; hi[0] = o[n][2]; hi[1] = o[n][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * DV; idx += blockDim.x) {
        const int r = idx / DV, d = idx % DV;
        const bool with_sink = sink != nullptr && split == 0;
        float M = with_sink ? sink[h0 + r] : -INFINITY;
#pragma unroll
        for (int w = 0; w < BA_WARPS; ++w) M = fmaxf(M, s_m[w * 16 + r]);
        float L = with_sink ? expf(sink[h0 + r] - M) : 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < BA_WARPS; ++w) {
            const float f = s_m[w * 16 + r] == -INFINITY ? 0.f : expf(s_m[w * 16 + r] - M);
            L += s_l[w * 16 + r] * f;
            a += s_o[((size_t)w * 16 + r) * DV + d] * f;
        }
        if (n_splits == 1) {
            out[((size_t)t * nh + h0 + r) * DV + d] = __float2bfloat16_rn(a / L);
            continue;
        }
        float* dst = partial + (((size_t)t * nh + h0 + r) * n_splits + split) * (DV + 2);
        dst[2 + d] = a;
        if (d == 0) { dst[0] = M; dst[1] = L; }
    }
}

template <int DK, int DV>
int launch_bias_heads(const void* q, const void* cache, const float* bias_t, int far, const float* sink, const int* positions,
                      const int* seq_of_token, const int* page_table, int table_stride, int page_size, int window,
                      int keep_first, int cell, float scale, float softcap, void* out, float* partial, int n_splits, int T_, int nh, int nkv,
                      int n_seqs, int n_pages, cudaStream_t stream) {
    auto kern = bias_attention_heads_kernel<DK, DV>;
    const int ring = BA_WARPS * 2 * BH_K * (DK + DV + 8) * (int)sizeof(__nv_bfloat16);
    const int merge = (BA_WARPS * 16 * 2 + BA_WARPS * 16 * DV) * (int)sizeof(float);
    const int smem = ring > merge ? ring : merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) TQ_FAIL(-1, "bias_attention_heads: %d bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int chunks = (nh / nkv + 15) / 16;
    dim3 grid(T_, nkv * chunks, n_splits);
    tq_launch(grid, BA_WARPS * 32, smem, stream)(kern, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, bias_t, far, sink,
        positions, seq_of_token, page_table, table_stride, page_size, window, keep_first, cell, scale, softcap, (__nv_bfloat16*)out, partial,
        n_splits, nh, nkv, n_seqs, n_pages);
    return 0;
}

TQ_EXPORT int tq_bias_attention_heads(const void* q, const void* cache, const float* bias_t, int far, const float* sink,
                                      const int* positions, const int* seq_of_token, const int* page_table,
                                      int table_stride, int page_size, int window, int keep_first, int cell, float scale, float softcap, void* out,
                                      float* partial, int n_splits, int T_, int nh, int nkv, int dk, int dv, int n_seqs,
                                      int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "bias_attention_heads: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE(page_size % BH_K == 0, "bias_attention_heads: pages of %d positions are no multiple of %d", page_size, BH_K);
    TQ_REQUIRE(window >= 0 && keep_first >= 0 && far >= 0, "bias_attention_heads: negative window, kept positions or distance");
    TQ_REQUIRE(n_splits >= 1 && n_splits <= 65535 && (long long)nkv * ((nh / nkv + 15) / 16) <= 65535,
               "bias_attention_heads: %d ranges or %d key/value heads exceed the grid limit", n_splits, nkv);
    TQ_REQUIRE(n_splits == 1 || partial != nullptr, "bias_attention_heads: %d ranges need scratch for their states", n_splits);
    int rc = -2;
#define BH_CASE(DK_, DV_) if (dk == DK_ && dv == DV_) rc = launch_bias_heads<DK_, DV_>(q, cache, bias_t, far, sink, positions, \
        seq_of_token, page_table, table_stride, page_size, window, keep_first, cell, scale, softcap, out, partial, n_splits, T_, nh, nkv,  \
        n_seqs, n_pages, stream);
    BH_CASE(32, 32) BH_CASE(32, 64) BH_CASE(32, 128) BH_CASE(64, 32) BH_CASE(64, 64) BH_CASE(64, 128)
    BH_CASE(128, 32) BH_CASE(128, 64) BH_CASE(128, 128)
#undef BH_CASE
    TQ_REQUIRE(rc != -2, "bias_attention_heads: key size %d and value size %d must each be 32, 64 or 128", dk, dv);
    if (rc) return rc;
    TQ_CHECK_LAUNCH("bias_attention_heads");
    if (n_splits > 1) {
        tq_launch(T_ * nh, dv >= 128 ? 128 : 64, 0, stream)(bias_attention_merge_kernel<__nv_bfloat16>, partial, n_splits, dv, (__nv_bfloat16*)out);
        TQ_CHECK_LAUNCH("bias_attention_merge");
    }
    return 0;
}

template <int DK, int DV>
int launch_bias_runs(const void* q, const void* cache, const float* bias_t, int far, const float* sink,
                     const int* cu_seqlens, const int* seq_start, const int* page_table, int table_stride, int window,
                     int keep_first, int cell, float scale, float softcap, void* out, int n_seqs, int max_run, int nh, int nkv, int n_pages,
                     cudaStream_t stream) {
    auto kern = bias_attention_runs_kernel<DK, DV>;
    const int smem = 2 * BR_K * (DK + DV + 8) * (int)sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) TQ_FAIL(-1, "bias_attention_runs: %d bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(nh, n_seqs, (max_run + BR_Q - 1) / BR_Q);
    tq_launch(grid, BR_WARPS * 32, smem, stream)(kern, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, bias_t, far,
        sink, cu_seqlens, seq_start, page_table, table_stride, window, keep_first, cell, scale, softcap, (__nv_bfloat16*)out, nh, nkv, n_pages);
    return 0;
}

// bias_t: the bias per head and distance, [heads][far + 1] (the transpose of what tq_bias_attention takes).
TQ_EXPORT int tq_bias_attention_runs(const void* q, const void* cache, int act_dtype, const float* bias_t, int far,
                                     const float* sink, const int* cu_seqlens, const int* seq_start,
                                     const int* page_table, int table_stride, int page_size, int window,
                                     int keep_first, int cell, float scale, float softcap, void* out, int n_seqs, int max_run, int nh, int nkv,
                                     int dk, int dv, int n_pages, cudaStream_t stream) {
    if (n_seqs == 0 || max_run == 0) return 0;
    TQ_REQUIRE(act_dtype == TQ_BF16, "bias_attention_runs: bfloat16 only");
    TQ_REQUIRE(page_size == BR_K, "bias_attention_runs: pages of %d positions, not %d", BR_K, page_size);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "bias_attention_runs: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE(n_seqs <= 65535 && (max_run + BR_Q - 1) / BR_Q <= 65535, "bias_attention_runs: %d sequences or runs of %d tokens exceed the grid limit", n_seqs, max_run);
    TQ_REQUIRE(window >= 0 && keep_first >= 0 && far >= 0, "bias_attention_runs: negative window, kept positions or distance");
    int rc = -2;
#define BR_CASE(DK_, DV_) if (dk == DK_ && dv == DV_) rc = launch_bias_runs<DK_, DV_>(q, cache, bias_t, far, sink, cu_seqlens, \
        seq_start, page_table, table_stride, window, keep_first, cell, scale, softcap, out, n_seqs, max_run, nh, nkv, n_pages, stream);
    BR_CASE(32, 32) BR_CASE(32, 64) BR_CASE(32, 128) BR_CASE(64, 32) BR_CASE(64, 64) BR_CASE(64, 128)
    BR_CASE(128, 32) BR_CASE(128, 64) BR_CASE(128, 128)
#undef BR_CASE
    TQ_REQUIRE(rc != -2, "bias_attention_runs: key size %d and value size %d must each be 32, 64 or 128", dk, dv);
    if (rc) return rc;
    TQ_CHECK_LAUNCH("bias_attention_runs");
    return 0;
}
