// Row-wise kernels: embedding rows, RMSNorm (with the residual sum and a row gather fused in),
// SiLU(gate)*up, row gather.  All statistics and the residual sum are computed in fp32.
//
// Formulas as the reference computes them on the CPU:
//   embedding  x = table[token]                       src/engine/tq_transformer.c:2298-2329
//   rmsnorm    ss = sum(x^2)/n + eps; y = x*(1/sqrt(ss))*w   src/engine/tq_ops.c:1373-1410
//   silu       x/(1+exp(-x))                          src/engine/tq_ops.c:1454-1478
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

// ---------------------------------------------------------------------------------------
// x[t, :] = table[tokens[t], :]  (fp32 residual stream out)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                  float* __restrict__ x, int H, int V) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const TW* row = table + (size_t)TQ_CHECKED(tokens[t], V, TQ_IDX_TOKEN) * H;
    float* out = x + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = tq_to_float(row[i]);
}

TQ_EXPORT int tq_embed_rows(const int* tokens, const void* table, int table_dtype, float* x,
                            int T, int H, int V, cudaStream_t stream) {
    if (T == 0) return 0;
    TQ_REQUIRE(T > 0 && H > 0, "embed_rows: bad sizes T=%d H=%d", T, H);
    const int threads = H >= 1024 ? 256 : 128;
    TQ_DISPATCH(table_dtype, TW,
        tq_launch(T, threads, 0, stream)(embed_rows_kernel<TW>, tokens, (const TW*)table, x, H, V));
    TQ_CHECK_LAUNCH("embed_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------
// RMSNorm over rows of the fp32 residual stream.
//   y given:    the norm is taken of x + y (the residual sum, in fp32)
//   rows given: the norm of row rows[r] is written to out[r] and x is not changed;
//               otherwise row r goes to out[r] and, with y, the sum is written back into x
// ---------------------------------------------------------------------------------------
template <typename TY, typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TY* __restrict__ y, const int* __restrict__ rows,
                               const TW* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + src * H;
    const TY* yr = y ? y + src * H : nullptr;
    const bool write_back = y && !rows;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (yr) v += tq_to_float(yr[i]);
        if (write_back) xr[i] = v;
        ss += v * v;
    }
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (yr && !write_back) v += tq_to_float(yr[i]);
        o[i] = tq_from_float<TO>(v * rs * tq_to_float(w[i]));
    }
}

// The same with 16-byte accesses: a thread keeps up to 8 groups of 4 elements of its row in registers
// between the two passes (H a multiple of 4, at most 32 * blockDim elements).
template <typename T> __device__ __forceinline__ float4 tq_load4(const T* p);
template <> __device__ __forceinline__ float4 tq_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 tq_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void tq_store4(T* p, float4 v);
template <> __device__ __forceinline__ void tq_store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void tq_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

#define RMS_VEC_GROUPS 8
template <typename TY, typename TW, typename TO>
__global__ void rmsnorm_vec_kernel(float* __restrict__ x, const TY* __restrict__ y, const int* __restrict__ rows,
                                   const TW* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + src * H;
    const TY* yr = y ? y + src * H : nullptr;
    const bool write_back = y && !rows;
    const int nvec = H >> 2;
    float4 v[RMS_VEC_GROUPS], g[RMS_VEC_GROUPS];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < RMS_VEC_GROUPS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            g[c] = tq_load4<TW>(w + 4 * i);                 // fetched now, so that it arrives during the reduction
            float4 a = tq_load4<float>(xr + 4 * i);
            if (yr) { const float4 b = tq_load4<TY>(yr + 4 * i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
            if (write_back) tq_store4<float>(xr + 4 * i, a);
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            v[c] = a;
        }
    }
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
#pragma unroll
    for (int c = 0; c < RMS_VEC_GROUPS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec)
            tq_store4<TO>(o + 4 * i, make_float4(v[c].x * rs * g[c].x, v[c].y * rs * g[c].y, v[c].z * rs * g[c].z,
                                                 v[c].w * rs * g[c].w));
    }
}

// Many rows (prompts): a warp per row, the row in registers (up to 16 groups of 4 elements per lane: H <= 2048, a
// multiple of 4), the sums by shuffles: no block-wide barrier, and a lane's loads are all in flight together.
#define RMS_WARP_GROUPS 16
#define RMS_WARP_ROWS 8          // warps (rows) per block
template <typename TY, typename TW, typename TO>
__global__ void __launch_bounds__(32 * RMS_WARP_ROWS)
rmsnorm_warp_kernel(float* __restrict__ x, const TY* __restrict__ y, const int* __restrict__ rows,
                    const TW* __restrict__ w, TO* __restrict__ out, int R, int H, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * RMS_WARP_ROWS + (threadIdx.x >> 5);
    if (r >= R) return;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + src * H;
    const TY* yr = y ? y + src * H : nullptr;
    const bool write_back = y && !rows;
    const int nvec = H >> 2;
    float4 v[RMS_WARP_GROUPS];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
        const int i = lane + 32 * c;
        if (i < nvec) v[c] = tq_load4<float>(xr + 4 * i);
    }
    if (yr) {
#pragma unroll
        for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
            const int i = lane + 32 * c;
            if (i < nvec) { const float4 b = tq_load4<TY>(yr + 4 * i); v[c].x += b.x; v[c].y += b.y; v[c].z += b.z; v[c].w += b.w; }
        }
    }
#pragma unroll
    for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
        const int i = lane + 32 * c;
        if (i < nvec) {
            if (write_back) tq_store4<float>(xr + 4 * i, v[c]);
            ss += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
        }
    }
    ss = tq_warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
#pragma unroll
    for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
        const int i = lane + 32 * c;
        if (i < nvec) {
            const float4 g = tq_load4<TW>(w + 4 * i);
            tq_store4<TO>(o + 4 * i, make_float4(v[c].x * rs * g.x, v[c].y * rs * g.y, v[c].z * rs * g.z, v[c].w * rs * g.w));
        }
    }
}

TQ_EXPORT int tq_rmsnorm(float* x, const void* y, int y_dtype, const int* rows, const void* w, int w_dtype,
                         void* out, int out_dtype, int R, int H, float eps, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && H > 0, "rmsnorm: bad sizes R=%d H=%d", R, H);
    if (H % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
        ((uintptr_t)out % 16) == 0) {
        if (R >= 512 && H / 4 <= 32 * RMS_WARP_GROUPS) {
            TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
                (tq_launch((R + RMS_WARP_ROWS - 1) / RMS_WARP_ROWS, 32 * RMS_WARP_ROWS, 0, stream)(
                    rmsnorm_warp_kernel<TY, TW, TO>, x, (const TY*)y, rows, (const TW*)w, (TO*)out, R, H, eps)))));
            TQ_CHECK_LAUNCH("rmsnorm");
            return 0;
        }
        int vthreads = ((H / 4 + 31) / 32) * 32;
        if (vthreads > 256 && H / 4 <= 256 * RMS_VEC_GROUPS) vthreads = ((H / 4 + 255) / 256 <= 4) ? 256 : 512;
        if (vthreads > 1024) vthreads = 1024;
        if (H / 4 <= vthreads * RMS_VEC_GROUPS) {
            TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
                (tq_launch(R, vthreads, 0, stream)(rmsnorm_vec_kernel<TY, TW, TO>, x, (const TY*)y, rows, (const TW*)w,
                                                                            (TO*)out, H, eps)))));
            TQ_CHECK_LAUNCH("rmsnorm");
            return 0;
        }
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
        (tq_launch(R, threads, 0, stream)(rmsnorm_kernel<TY, TW, TO>, x, (const TY*)y, rows, (const TW*)w,
                                                              (TO*)out, H, eps)))));
    TQ_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------------------
// x[r] += y[r]  (fp32 residual stream; used where no norm follows the sum)
// ---------------------------------------------------------------------------------------
template <typename TY>
__global__ void residual_add_kernel(float* __restrict__ x, const TY* __restrict__ y, size_t n) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] += tq_to_float(y[i]);
}

TQ_EXPORT int tq_residual_add(float* x, const void* y, int y_dtype, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    TQ_DISPATCH(y_dtype, TY,
        tq_launch((int)blocks, threads, 0, stream)(residual_add_kernel<TY>, x, (const TY*)y, (size_t)n));
    TQ_CHECK_LAUNCH("residual_add");
    return 0;
}

// ---------------------------------------------------------------------------------------
// x[t, i] += bias[i], in place, summed in fp32 (for a projection whose bias no fused kernel adds)
// ---------------------------------------------------------------------------------------
template <typename TX, typename TB>
__global__ void add_bias_kernel(TX* __restrict__ x, const TB* __restrict__ bias, int N) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    TX* row = x + (size_t)blockIdx.x * N;
    for (int i = threadIdx.x; i < N; i += blockDim.x)
        row[i] = tq_from_float<TX>(tq_to_float(row[i]) + tq_to_float(bias[i]));
}

TQ_EXPORT int tq_add_bias(void* x, int x_dtype, const void* bias, int bias_dtype, int T_, int N, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ > 0 && N > 0, "add_bias: bad sizes T=%d N=%d", T_, N);
    TQ_DISPATCH(x_dtype, TX, TQ_DISPATCH(bias_dtype, TB,
        (tq_launch(T_, 256, 0, stream)(add_bias_kernel<TX, TB>, (TX*)x, (const TB*)bias, N))));
    TQ_CHECK_LAUNCH("add_bias");
    return 0;
}

// ---------------------------------------------------------------------------------------
// h[t, i] = glu(gu[t, i], gu[t, I + i])   (gate rows first, then up rows; glu: common.cuh, silu(gate) * up by default)
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ gu, TO* __restrict__ h, int I, TqGlu act) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const TI* g = gu + (size_t)t * 2 * I;
    TO* o = h + (size_t)t * I;
    for (int i = threadIdx.x; i < I; i += blockDim.x) {
        const float a = tq_to_float(g[i]), b = tq_to_float(g[I + i]);
        o[i] = tq_from_float<TO>(tq_glu(a, b, act));
    }
}

// limit <= 0: no caps.  (limit, slope, offset) = (0, 1, 0): silu(gate) * up.
TQ_EXPORT int tq_glu_mul(const void* gu, int in_dtype, void* h, int out_dtype, int T_, int I, float limit, float slope,
                         float offset, int kind, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ > 0 && I > 0, "glu_mul: bad sizes T=%d I=%d", T_, I);
    TQ_REQUIRE(kind == TQ_GLU_SIGMOID || kind == TQ_GLU_GELU_TANH, "glu_mul: unknown activation kind %d", kind);
    const TqGlu act = tq_glu_params(limit, slope, offset, kind);
    TQ_DISPATCH(in_dtype, TI, TQ_DISPATCH(out_dtype, TO,
        (tq_launch(T_, 256, 0, stream)(silu_mul_kernel<TI, TO>, (const TI*)gu, (TO*)h, I, act))));
    TQ_CHECK_LAUNCH("glu_mul");
    return 0;
}

TQ_EXPORT int tq_silu_mul(const void* gu, int in_dtype, void* h, int out_dtype, int T_, int I, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ > 0 && I > 0, "silu_mul: bad sizes T=%d I=%d", T_, I);
    const TqGlu act = tq_glu_params(0.f, 1.f, 0.f);
    TQ_DISPATCH(in_dtype, TI, TQ_DISPATCH(out_dtype, TO,
        (tq_launch(T_, 256, 0, stream)(silu_mul_kernel<TI, TO>, (const TI*)gu, (TO*)h, I, act))));
    TQ_CHECK_LAUNCH("silu_mul");
    return 0;
}

// ---------------------------------------------------------------------------------------
// out[r, :] = in[idx[r] / divisor, :]   (expert-sorted copies of token rows: divisor = top-k)
// ---------------------------------------------------------------------------------------
// A warp copies a row (16-byte accesses when rows allow it); a block takes several rows.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ in, const int* __restrict__ idx, int divisor,
                                   T* __restrict__ out, int R, int H, int vec, int S) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < R; r += gridDim.x * warps) {
        const T* src = in + (size_t)TQ_CHECKED(idx[r] / divisor, S, TQ_IDX_ROW) * H;
        T* dst = out + (size_t)r * H;
        if (vec) {          // rows are a multiple of 16 bytes and 16-byte aligned
            const int n16 = (int)((size_t)H * sizeof(T) / 16);
            const uint4* s4 = reinterpret_cast<const uint4*>(src);
            uint4* d4 = reinterpret_cast<uint4*>(dst);
            for (int i0 = lane; i0 < n16; i0 += 256) {      // eight 16-byte loads in flight per lane, then the stores
                uint4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) if (i0 + 32 * j < n16) v[j] = s4[i0 + 32 * j];
#pragma unroll
                for (int j = 0; j < 8; ++j) if (i0 + 32 * j < n16) d4[i0 + 32 * j] = v[j];
            }
        } else {
            for (int i = lane; i < H; i += 32) dst[i] = src[i];
        }
    }
}

// S: rows of `in` (what the indices are checked against in a debug build).
TQ_EXPORT int tq_gather_rows(const void* in, const int* idx, int divisor, void* out, int dtype, int R, int H, int S,
                             cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && H > 0 && divisor > 0, "gather_rows: bad sizes R=%d H=%d divisor=%d", R, H, divisor);
    const int esize = dtype == TQ_F32 ? 4 : 2;
    const int vec = ((size_t)H * esize) % 16 == 0 && ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0;
    int blocks = (R + 7) / 8;                     // eight warps, a row each, per block
    if (blocks > 148 * 8) blocks = 148 * 8;
    TQ_DISPATCH(dtype, T,
        tq_launch(blocks, 256, 0, stream)(gather_rows_kernel<T>, (const T*)in, idx, divisor, (T*)out, R, H, vec, S));
    TQ_CHECK_LAUNCH("gather_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Embedding with a scale and a table of token pairs:
//   x[t] = table[tok] * scale + pair[(prev * mul_prev + tok * mul_cur) mod buckets]
// where prev is the token before tok in its sequence; a sequence's first token takes the pair table's row
// `buckets`.  The token before a step's first token comes from last_token[slot], the sequence's state; the block
// of a sequence's first token of the step reads it and then stores the step's last token there (one thread, read
// before write, and no other block touches that slot).  pair == nullptr: no pair table, no state.
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_pair_rows_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                       const TW* __restrict__ pair, float* __restrict__ x, int H, int V, float scale,
                                       int buckets, long long mul_prev, long long mul_cur,
                                       const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                                       const int* __restrict__ seq_start, const int* __restrict__ slots,
                                       int* __restrict__ last_token, int n_seqs) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ int s_row;
    const int t = blockIdx.x;
    const int tok = TQ_CHECKED(tokens[t], V, TQ_IDX_TOKEN);
    if (pair && threadIdx.x == 0) {
        const int s = TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE);
        const int first = cu_seqlens[s];
        long long prev = -1;
        if (t > first) {
            prev = tokens[t - 1];
        } else {
            if (seq_start[s] > 0) prev = last_token[slots[s]];
            last_token[slots[s]] = tokens[cu_seqlens[s + 1] - 1];
        }
        long long r = buckets;
        if (prev >= 0) {
            r = (prev * mul_prev + (long long)tok * mul_cur) % buckets;
            if (r < 0) r += buckets;
        }
        s_row = (int)r;
    }
    __syncthreads();
    const TW* row = table + (size_t)tok * H;
    const TW* prow = pair ? pair + (size_t)s_row * H : nullptr;
    float* out = x + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = tq_to_float(row[i]) * scale;
        if (prow) v += tq_to_float(prow[i]);
        out[i] = v;
    }
}

TQ_EXPORT int tq_embed_pair_rows(const int* tokens, const void* table, const void* pair, int table_dtype, float* x,
                                 int T_, int H, int V, float scale, int buckets, long long mul_prev, long long mul_cur,
                                 const int* seq_of_token, const int* cu_seqlens, const int* seq_start, const int* slots,
                                 int* last_token, int n_seqs, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ > 0 && H > 0, "embed_pair_rows: bad sizes T=%d H=%d", T_, H);
    TQ_REQUIRE(!pair || (buckets > 0 && last_token), "embed_pair_rows: a pair table needs buckets and a state");
    const int threads = H >= 1024 ? 256 : 128;
    TQ_DISPATCH(table_dtype, TW,
        tq_launch(T_, threads, 0, stream)(embed_pair_rows_kernel<TW>, tokens, (const TW*)table, (const TW*)pair, x, H, V,
                                          scale, buckets, mul_prev, mul_cur, seq_of_token, cu_seqlens, seq_start, slots,
                                          last_token, n_seqs));
    TQ_CHECK_LAUNCH("embed_pair_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Residual sum with the norm on the sub-layer's output: x[r] += y[r] / sqrt(mean(y[r]^2) + eps) * w, in fp32;
// `copy` (optional) receives the new x in the activation dtype for the products that read it next.
// ---------------------------------------------------------------------------------------
template <typename TY, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TY* __restrict__ y, const TW* __restrict__ w,
                                   TO* __restrict__ copy, int H, float eps, const TW* __restrict__ next_w,
                                   TO* __restrict__ next_out, float next_eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    const TY* yr = y + r * H;
    float* xr = x + r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = tq_to_float(yr[i]);
        ss += v * v;
    }
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = xr[i] + tq_to_float(yr[i]) * rs * tq_to_float(w[i]);
        xr[i] = v;
        s2 += v * v;
        if (copy) copy[r * H + i] = tq_from_float<TO>(v);
    }
    if (next_out == nullptr) return;               // the same for the whole block
    s2 = tq_block_sum(s2, scratch);
    const float rs2 = 1.0f / sqrtf(s2 / (float)H + next_eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)      // a thread reads back what it wrote itself
        next_out[r * H + i] = tq_from_float<TO>(xr[i] * rs2 * tq_to_float(next_w[i]));
}

// The same for float32 y in rows of up to 4 * ADDN_THREADS * NV elements, a multiple of four: a thread keeps its
// float4 pieces of y in registers between the sum of squares and the update, so y is read once.
#define ADDN_THREADS 256
template <typename TW, typename TO, int NV>
__global__ void __launch_bounds__(ADDN_THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const TW* __restrict__ w,
                       TO* __restrict__ copy, int H, float eps, const TW* __restrict__ next_w,
                       TO* __restrict__ next_out, float next_eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    const float4* yr = reinterpret_cast<const float4*>(y + r * H);
    float4* xr = reinterpret_cast<float4*>(x + r * H);
    const int n4 = H / 4;
    float4 yv[NV], xv[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * ADDN_THREADS;
        yv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            yv[k] = yr[i];
            xv[k] = xr[i];
        }
        ss += yv[k].x * yv[k].x + yv[k].y * yv[k].y + yv[k].z * yv[k].z + yv[k].w * yv[k].w;
    }
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * ADDN_THREADS;
        if (i < n4) {
            float4 v;
            v.x = xv[k].x + yv[k].x * rs * tq_to_float(w[4 * i]);
            v.y = xv[k].y + yv[k].y * rs * tq_to_float(w[4 * i + 1]);
            v.z = xv[k].z + yv[k].z * rs * tq_to_float(w[4 * i + 2]);
            v.w = xv[k].w + yv[k].w * rs * tq_to_float(w[4 * i + 3]);
            xr[i] = v;
            xv[k] = v;
            s2 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            if (copy) {
                TO* c = copy + r * H + 4 * i;
                c[0] = tq_from_float<TO>(v.x); c[1] = tq_from_float<TO>(v.y);
                c[2] = tq_from_float<TO>(v.z); c[3] = tq_from_float<TO>(v.w);
            }
        }
    }
    if (next_out == nullptr) return;               // the same for the whole block
    s2 = tq_block_sum(s2, scratch);
    const float rs2 = 1.0f / sqrtf(s2 / (float)H + next_eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * ADDN_THREADS;
        if (i < n4) {
            TO* c = next_out + r * H + 4 * i;
            c[0] = tq_from_float<TO>(xv[k].x * rs2 * tq_to_float(next_w[4 * i]));
            c[1] = tq_from_float<TO>(xv[k].y * rs2 * tq_to_float(next_w[4 * i + 1]));
            c[2] = tq_from_float<TO>(xv[k].z * rs2 * tq_to_float(next_w[4 * i + 2]));
            c[3] = tq_from_float<TO>(xv[k].w * rs2 * tq_to_float(next_w[4 * i + 3]));
        }
    }
}

// next_w, next_out (optional, in the dtypes of w and of copy): the norm that reads the new x next,
// next_out[r] = x[r] / sqrt(mean(x[r]^2) + next_eps) * next_w, taken in the same pass.
TQ_EXPORT int tq_add_rmsnorm(float* x, const void* y, int y_dtype, const void* w, int w_dtype, void* copy,
                             int copy_dtype, int R, int H, float eps, const void* next_w, void* next_out, float next_eps,
                             cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && H > 0, "add_rmsnorm: bad sizes R=%d H=%d", R, H);
    TQ_REQUIRE(next_out == nullptr || next_w != nullptr, "add_rmsnorm: a following norm without its weight%s", "");
    if (y_dtype == TQ_F32 && H % 4 == 0 && H <= 4 * ADDN_THREADS * 4 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0) {
        const int nv = (H / 4 + ADDN_THREADS - 1) / ADDN_THREADS;
#define ADDN_LAUNCH(NV_)                                                                                           \
        TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(copy_dtype, TO,                                                       \
            (tq_launch(R, ADDN_THREADS, 0, stream)(add_rmsnorm_vec_kernel<TW, TO, NV_>, x, (const float*)y, (const TW*)w, \
                                                   (TO*)copy, H, eps, (const TW*)next_w, (TO*)next_out, next_eps))))
        if (nv <= 1) ADDN_LAUNCH(1);
        else if (nv == 2) ADDN_LAUNCH(2);
        else ADDN_LAUNCH(4);
#undef ADDN_LAUNCH
        TQ_CHECK_LAUNCH("add_rmsnorm");
        return 0;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(copy_dtype, TO,
        (tq_launch(R, threads, 0, stream)(add_rmsnorm_kernel<TY, TW, TO>, x, (const TY*)y, (const TW*)w, (TO*)copy, H,
                                          eps, (const TW*)next_w, (TO*)next_out, next_eps)))));
    TQ_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------------------
// out[i] = act(in[i]) elementwise; act 0: identity (a change of dtype), 1: the square of relu
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void map_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n, int act) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float v = tq_to_float(in[i]);
        if (act == 1) { v = fmaxf(v, 0.f); v = v * v; }
        out[i] = tq_from_float<TO>(v);
    }
}

TQ_EXPORT int tq_map(const void* in, int in_dtype, void* out, int out_dtype, long long n, int act, cudaStream_t stream) {
    if (n == 0) return 0;
    TQ_REQUIRE(act == 0 || act == 1, "map: unknown function %d", act);
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    TQ_DISPATCH(in_dtype, TI, TQ_DISPATCH(out_dtype, TO,
        (tq_launch((int)blocks, threads, 0, stream)(map_kernel<TI, TO>, (const TI*)in, (TO*)out, (size_t)n, act))));
    TQ_CHECK_LAUNCH("map");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Rotation of interleaved pairs in place: rows [T, heads, row] (row stride given), the pairs (2i, 2i+1) of the
// `n_pairs` first pairs from element `offset` of each head turn by angle = position * freq[i]; cos and sin carry the
// factor `mag`.  Angles in fp32.
// ---------------------------------------------------------------------------------------
template <typename TX>
__global__ void rotate_pairs_kernel(TX* __restrict__ x, const float* __restrict__ freq, const int* __restrict__ positions,
                                    int heads, int head_stride, long long token_stride, int offset, int n_pairs, float mag) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    for (int k = threadIdx.x; k < heads * n_pairs; k += blockDim.x) {
        const int h = k / n_pairs, i = k % n_pairs;
        float s, c;
        sincosf(pos * freq[i], &s, &c);
        s *= mag; c *= mag;
        TX* p = x + (size_t)t * token_stride + (size_t)h * head_stride + offset + 2 * i;
        const float u = tq_to_float(p[0]), v = tq_to_float(p[1]);
        p[0] = tq_from_float<TX>(u * c - v * s);
        p[1] = tq_from_float<TX>(v * c + u * s);
    }
}

TQ_EXPORT int tq_rotate_pairs(void* x, int dtype, const float* freq, const int* positions, int T_, int heads,
                              int head_stride, long long token_stride, int offset, int n_pairs, float mag,
                              cudaStream_t stream) {
    if (T_ == 0 || n_pairs == 0 || heads == 0) return 0;
    TQ_REQUIRE(T_ > 0 && heads > 0 && n_pairs > 0 && offset >= 0, "rotate_pairs: bad sizes");
    TQ_DISPATCH(dtype, TX,
        tq_launch(T_, 128, 0, stream)(rotate_pairs_kernel<TX>, (TX*)x, freq, positions, heads, head_stride, token_stride,
                                      offset, n_pairs, mag));
    TQ_CHECK_LAUNCH("rotate_pairs");
    return 0;
}

// ---------------------------------------------------------------------------------------
// The mean of two branches, each under an RMS norm of its own:
//   out[r] = (a[r] / sqrt(mean(a[r]^2) + eps) * wa + b[r] / sqrt(mean(b[r]^2) + eps) * wb) / 2, in fp32.
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void mean_of_norms_kernel(const float* __restrict__ a, const TW* __restrict__ wa, const float* __restrict__ b,
                                     const TW* __restrict__ wb, float* __restrict__ out, int H, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    const float* ar = a + r * H;
    const float* br = b + r * H;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float u = ar[i], v = br[i];
        sa += u * u;
        sb += v * v;
    }
    sa = tq_block_sum(sa, scratch);
    sb = tq_block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)H + eps), rb = 1.0f / sqrtf(sb / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[r * H + i] = 0.5f * (ar[i] * ra * tq_to_float(wa[i]) + br[i] * rb * tq_to_float(wb[i]));
}

TQ_EXPORT int tq_mean_of_norms(const float* a, const void* wa, const float* b, const void* wb, int w_dtype, float* out,
                               int R, int H, float eps, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && H > 0, "mean_of_norms: bad sizes R=%d H=%d", R, H);
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    TQ_DISPATCH(w_dtype, TW,
        (tq_launch(R, threads, 0, stream)(mean_of_norms_kernel<TW>, a, (const TW*)wa, b, (const TW*)wb, out, H, eps)));
    TQ_CHECK_LAUNCH("mean_of_norms");
    return 0;
}

// ---------------------------------------------------------------------------------------
// The mean of two normed branches under a further norm, summed into the stream, with the norm that reads the stream
// next (optional) in the same pass:
//   m[r] = (a[r] / sqrt(mean(a[r]^2) + pair_eps) * wa + b[r] / sqrt(mean(b[r]^2) + pair_eps) * wb) / 2
//   x[r] += m[r] / sqrt(mean(m[r]^2) + eps) * w;   next_out[r] = x[r] / sqrt(mean(x[r]^2) + next_eps) * next_w
// all in fp32.  The vector form keeps a thread's float4 pieces of the row in registers from the first sums to the last
// output (rows of a multiple of four, up to 4 * ADDN_THREADS * NV elements); the plain form reads the row again.
// ---------------------------------------------------------------------------------------
template <typename TW, typename TO, int NV>
__global__ void __launch_bounds__(ADDN_THREADS)
add_rmsnorm_pair_vec_kernel(float* __restrict__ x, const float* __restrict__ a, const TW* __restrict__ wa,
                            const float* __restrict__ b, const TW* __restrict__ wb, float pair_eps,
                            const TW* __restrict__ w, TO* __restrict__ copy, int H, float eps,
                            const TW* __restrict__ next_w, TO* __restrict__ next_out, float next_eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    const float4* ar = reinterpret_cast<const float4*>(a + r * H);
    const float4* br = reinterpret_cast<const float4*>(b + r * H);
    float4* xr = reinterpret_cast<float4*>(x + r * H);
    const int n4 = H / 4;
    float4 av[NV], bv[NV], xv[NV];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * ADDN_THREADS;
        av[k] = bv[k] = xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            av[k] = ar[i];
            bv[k] = br[i];
            xv[k] = xr[i];
        }
        sa += av[k].x * av[k].x + av[k].y * av[k].y + av[k].z * av[k].z + av[k].w * av[k].w;
        sb += bv[k].x * bv[k].x + bv[k].y * bv[k].y + bv[k].z * bv[k].z + bv[k].w * bv[k].w;
    }
    sa = tq_block_sum(sa, scratch);
    sb = tq_block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)H + pair_eps), rb = 1.0f / sqrtf(sb / (float)H + pair_eps);
    float sm = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * ADDN_THREADS;
        if (i < n4) {
            float4 m;
            m.x = 0.5f * (av[k].x * ra * tq_to_float(wa[4 * i]) + bv[k].x * rb * tq_to_float(wb[4 * i]));
            m.y = 0.5f * (av[k].y * ra * tq_to_float(wa[4 * i + 1]) + bv[k].y * rb * tq_to_float(wb[4 * i + 1]));
            m.z = 0.5f * (av[k].z * ra * tq_to_float(wa[4 * i + 2]) + bv[k].z * rb * tq_to_float(wb[4 * i + 2]));
            m.w = 0.5f * (av[k].w * ra * tq_to_float(wa[4 * i + 3]) + bv[k].w * rb * tq_to_float(wb[4 * i + 3]));
            av[k] = m;
            sm += m.x * m.x + m.y * m.y + m.z * m.z + m.w * m.w;
        }
    }
    sm = tq_block_sum(sm, scratch);
    const float rs = 1.0f / sqrtf(sm / (float)H + eps);
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * ADDN_THREADS;
        if (i < n4) {
            float4 v;
            v.x = xv[k].x + av[k].x * rs * tq_to_float(w[4 * i]);
            v.y = xv[k].y + av[k].y * rs * tq_to_float(w[4 * i + 1]);
            v.z = xv[k].z + av[k].z * rs * tq_to_float(w[4 * i + 2]);
            v.w = xv[k].w + av[k].w * rs * tq_to_float(w[4 * i + 3]);
            xr[i] = v;
            xv[k] = v;
            s2 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            if (copy) {
                TO* c = copy + r * H + 4 * i;
                c[0] = tq_from_float<TO>(v.x); c[1] = tq_from_float<TO>(v.y);
                c[2] = tq_from_float<TO>(v.z); c[3] = tq_from_float<TO>(v.w);
            }
        }
    }
    if (next_out == nullptr) return;               // the same for the whole block
    s2 = tq_block_sum(s2, scratch);
    const float rs2 = 1.0f / sqrtf(s2 / (float)H + next_eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * ADDN_THREADS;
        if (i < n4) {
            TO* c = next_out + r * H + 4 * i;
            c[0] = tq_from_float<TO>(xv[k].x * rs2 * tq_to_float(next_w[4 * i]));
            c[1] = tq_from_float<TO>(xv[k].y * rs2 * tq_to_float(next_w[4 * i + 1]));
            c[2] = tq_from_float<TO>(xv[k].z * rs2 * tq_to_float(next_w[4 * i + 2]));
            c[3] = tq_from_float<TO>(xv[k].w * rs2 * tq_to_float(next_w[4 * i + 3]));
        }
    }
}

template <typename TW, typename TO>
__global__ void add_rmsnorm_pair_kernel(float* __restrict__ x, const float* __restrict__ a, const TW* __restrict__ wa,
                                        const float* __restrict__ b, const TW* __restrict__ wb, float pair_eps,
                                        const TW* __restrict__ w, TO* __restrict__ copy, int H, float eps,
                                        const TW* __restrict__ next_w, TO* __restrict__ next_out, float next_eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    const float* ar = a + r * H;
    const float* br = b + r * H;
    float* xr = x + r * H;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        sa += ar[i] * ar[i];
        sb += br[i] * br[i];
    }
    sa = tq_block_sum(sa, scratch);
    sb = tq_block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)H + pair_eps), rb = 1.0f / sqrtf(sb / (float)H + pair_eps);
    auto mean = [&](int i) { return 0.5f * (ar[i] * ra * tq_to_float(wa[i]) + br[i] * rb * tq_to_float(wb[i])); };
    float sm = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float m = mean(i);
        sm += m * m;
    }
    sm = tq_block_sum(sm, scratch);
    const float rs = 1.0f / sqrtf(sm / (float)H + eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = xr[i] + mean(i) * rs * tq_to_float(w[i]);
        xr[i] = v;
        s2 += v * v;
        if (copy) copy[r * H + i] = tq_from_float<TO>(v);
    }
    if (next_out == nullptr) return;               // the same for the whole block
    s2 = tq_block_sum(s2, scratch);
    const float rs2 = 1.0f / sqrtf(s2 / (float)H + next_eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)      // a thread reads back what it wrote itself
        next_out[r * H + i] = tq_from_float<TO>(xr[i] * rs2 * tq_to_float(next_w[i]));
}

// wa, wb, w and next_w share one dtype; copy and next_out another.
TQ_EXPORT int tq_add_rmsnorm_pair(float* x, const float* a, const void* wa, const float* b, const void* wb, float pair_eps,
                                  const void* w, int w_dtype, void* copy, int copy_dtype, int R, int H, float eps,
                                  const void* next_w, void* next_out, float next_eps, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && H > 0, "add_rmsnorm_pair: bad sizes R=%d H=%d", R, H);
    TQ_REQUIRE(next_out == nullptr || next_w != nullptr, "add_rmsnorm_pair: a following norm without its weight%s", "");
    if (H % 4 == 0 && H <= 4 * ADDN_THREADS * 4 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0) {
        const int nv = (H / 4 + ADDN_THREADS - 1) / ADDN_THREADS;
#define ADDP_LAUNCH(NV_)                                                                                           \
        TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(copy_dtype, TO,                                                       \
            (tq_launch(R, ADDN_THREADS, 0, stream)(add_rmsnorm_pair_vec_kernel<TW, TO, NV_>, x, a, (const TW*)wa, b, \
                (const TW*)wb, pair_eps, (const TW*)w, (TO*)copy, H, eps, (const TW*)next_w, (TO*)next_out, next_eps))))
        if (nv <= 1) ADDP_LAUNCH(1);
        else if (nv == 2) ADDP_LAUNCH(2);
        else ADDP_LAUNCH(4);
#undef ADDP_LAUNCH
        TQ_CHECK_LAUNCH("add_rmsnorm_pair");
        return 0;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(copy_dtype, TO,
        (tq_launch(R, threads, 0, stream)(add_rmsnorm_pair_kernel<TW, TO>, x, a, (const TW*)wa, b, (const TW*)wb, pair_eps,
                                          (const TW*)w, (TO*)copy, H, eps, (const TW*)next_w, (TO*)next_out, next_eps))));
    TQ_CHECK_LAUNCH("add_rmsnorm_pair");
    return 0;
}

// ---------------------------------------------------------------------------------------
// A gated activation against rows of a table: out[t, j] = glu(z[t, j], table[tokens[t]][col0 + j]) for j < D
// (z fp32 [T, D]; the table's rows have `stride` elements).
// ---------------------------------------------------------------------------------------
template <typename TT, typename TO>
__global__ void glu_table_rows_kernel(const float* __restrict__ z, const int* __restrict__ tokens, const TT* __restrict__ table,
                                      int stride, int col0, TO* __restrict__ out, int D, int vocab, TqGlu act) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const size_t t = blockIdx.x;
    const TT* row = table + (size_t)TQ_CHECKED(tokens[t], vocab, TQ_IDX_TOKEN) * stride + col0;
    for (int j = threadIdx.x; j < D; j += blockDim.x)
        out[t * D + j] = tq_from_float<TO>(tq_glu(z[t * D + j], tq_to_float(row[j]), act));
}

TQ_EXPORT int tq_glu_table_rows(const float* z, const int* tokens, const void* table, int table_dtype, int stride, int col0,
                                void* out, int out_dtype, int T_, int D, int vocab, float limit, float slope, float offset,
                                int kind, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(D > 0 && col0 >= 0 && col0 + D <= stride, "glu_table_rows: columns %d..%d of rows of %d", col0, col0 + D, stride);
    TQ_REQUIRE(kind == TQ_GLU_SIGMOID || kind == TQ_GLU_GELU_TANH, "glu_table_rows: unknown activation kind %d", kind);
    const TqGlu act = tq_glu_params(limit, slope, offset, kind);
    const int threads = D >= 256 ? 256 : (D >= 64 ? 64 : 32);
    TQ_DISPATCH(table_dtype, TT, TQ_DISPATCH(out_dtype, TO,
        (tq_launch(T_, threads, 0, stream)(glu_table_rows_kernel<TT, TO>, z, tokens, (const TT*)table, stride, col0, (TO*)out, D,
                                           vocab, act))));
    TQ_CHECK_LAUNCH("glu_table_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------
// x[t, j] = x[t, j] * scale + bias[j] for j < N, rows of `stride` floats (bias may be null).  Grid (row, column chunks).
// ---------------------------------------------------------------------------------------
__global__ void scale_bias_cols_kernel(float* __restrict__ x, const float* __restrict__ bias, float scale, int N, int stride) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    float* row = x + (size_t)blockIdx.x * stride;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < N; j += gridDim.y * blockDim.x)
        row[j] = bias ? row[j] * scale + bias[j] : row[j] * scale;
}

TQ_EXPORT int tq_scale_bias_cols(float* x, const float* bias, float scale, int T_, int N, int stride, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(N > 0 && N <= stride, "scale_bias_cols: %d columns of rows of %d", N, stride);
    // a few rows of many columns (a head's logits) spread over blocks by columns as well: 2048 columns a block
    const int threads = N >= 1024 ? 256 : 128;
    tq_launch(dim3(T_, (N + 8 * threads - 1) / (8 * threads)), threads, 0, stream)(scale_bias_cols_kernel, x, bias, scale, N, stride);
    TQ_CHECK_LAUNCH("scale_bias_cols");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Dynamic tanh, a norm without statistics: out[r, i] = tanh(alpha * v[i]) * w[i] + b[i] with v the row rows[r] of x
// (all rows in order if rows is null), or x + scale * y where y is given (x then takes the sum, as in rmsnorm).
// With `shift`, the output is mixed with the token before: out = h + (h' - h) * shift[i], h' being the norm's
// unshifted output for the previous token of the sequence: the row above inside a run of new tokens, the sequence's
// kept row (state, fp32 [slots][H] with a row stride) for a run's first token, which is zero at a sequence's start.
// keep != 0 (steps in which every sequence brings one token): the token's own unshifted output becomes the kept row
// in the same pass; otherwise tq_dyt_keep_last does that in a launch of its own, since other blocks still read the
// old rows.  Shift and y exclude each other (the row above must not change under the kernel).
// ---------------------------------------------------------------------------------------
template <typename TY, typename TW, typename TO>
__global__ void dyt_kernel(float* __restrict__ x, const TY* __restrict__ y, float scale, const int* __restrict__ rows, float alpha,
                           const TW* __restrict__ w, const TW* __restrict__ b, TO* __restrict__ out, int H,
                           const TW* __restrict__ shift, float* __restrict__ state, long long slot_stride,
                           const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                           const int* __restrict__ slots, int keep) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const size_t r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : r;
    float* xr = x + src * H;
    const float* above = nullptr;      // the row of the token before, inside this step
    float* kept = nullptr;             // the sequence's kept row
    if (shift != nullptr) {
        const int s = seq_of_token[src];
        kept = state + (size_t)slots[s] * slot_stride;
        if ((int)src > cu_seqlens[s]) above = xr - H;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
        float v = xr[i];
        if (y != nullptr) {
            v += scale * tq_to_float(y[src * H + i]);
            if (rows == nullptr) xr[i] = v;
        }
        const float wi = tq_to_float(w[i]), bi = tq_to_float(b[i]);
        float h = tanhf(alpha * v) * wi + bi;
        if (shift != nullptr) {
            const float before = above ? tanhf(alpha * above[i]) * wi + bi : kept[i];
            if (keep) kept[i] = h;
            h += (before - h) * tq_to_float(shift[i]);
        }
        out[r * H + i] = tq_from_float<TO>(h);
    }
}

// The same with four neighbouring elements a thread (rows of a multiple of four elements, 16-byte aligned): every
// load of a thread's piece is in flight before the first tanhf.
template <typename TY, typename TW, typename TO>
__global__ void dyt_vec_kernel(float* __restrict__ x, const TY* __restrict__ y, float scale, const int* __restrict__ rows, float alpha,
                               const TW* __restrict__ w, const TW* __restrict__ b, TO* __restrict__ out, int H,
                               const TW* __restrict__ shift, float* __restrict__ state, long long slot_stride,
                               const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                               const int* __restrict__ slots, int keep) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const size_t r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : r;
    float* xr = x + src * H;
    const float* above = nullptr;
    float* kept = nullptr;
    if (shift != nullptr) {
        const int s = seq_of_token[src];
        kept = state + (size_t)slots[s] * slot_stride;
        if ((int)src > cu_seqlens[s]) above = xr - H;
    }
    auto norm4 = [alpha](float4 v, float4 wi, float4 bi) {
        return make_float4(tanhf(alpha * v.x) * wi.x + bi.x, tanhf(alpha * v.y) * wi.y + bi.y,
                           tanhf(alpha * v.z) * wi.z + bi.z, tanhf(alpha * v.w) * wi.w + bi.w);
    };
    for (int i = 4 * (blockIdx.y * blockDim.x + threadIdx.x); i < H; i += 4 * gridDim.y * blockDim.x) {
        float4 v = tq_load4<float>(xr + i);
        const float4 wi = tq_load4<TW>(w + i), bi = tq_load4<TW>(b + i);
        float4 before = make_float4(0.f, 0.f, 0.f, 0.f), sh = before;
        if (shift != nullptr) {
            before = tq_load4<float>((above ? above : kept) + i);
            sh = tq_load4<TW>(shift + i);
        }
        if (y != nullptr) {
            const float4 a = tq_load4<TY>(y + src * H + i);
            v.x += scale * a.x; v.y += scale * a.y; v.z += scale * a.z; v.w += scale * a.w;
            if (rows == nullptr) tq_store4<float>(xr + i, v);
        }
        float4 h = norm4(v, wi, bi);
        if (shift != nullptr) {
            if (above) before = norm4(before, wi, bi);
            if (keep) tq_store4<float>(kept + i, h);
            h.x += (before.x - h.x) * sh.x; h.y += (before.y - h.y) * sh.y;
            h.z += (before.z - h.z) * sh.z; h.w += (before.w - h.w) * sh.w;
        }
        tq_store4<TO>(out + r * H + i, h);
    }
}

// kept row of every sequence <- the unshifted norm of its last token of this step; grid (sequences, column chunks)
template <typename TW>
__global__ void dyt_keep_last_kernel(const float* __restrict__ x, float alpha, const TW* __restrict__ w, const TW* __restrict__ b,
                                     int H, float* __restrict__ state, long long slot_stride,
                                     const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int s = blockIdx.x;
    const int last = cu_seqlens[s + 1] - 1;
    if (last < cu_seqlens[s]) return;
    const float* xr = x + (size_t)last * H;
    float* kept = state + (size_t)slots[s] * slot_stride;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x)
        kept[i] = tanhf(alpha * xr[i]) * tq_to_float(w[i]) + tq_to_float(b[i]);
}

TQ_EXPORT int tq_dyt(float* x, const void* y, int y_dtype, float scale, const int* rows, float alpha, const void* w,
                     const void* b, int w_dtype, void* out, int out_dtype, int R, int H, const void* shift, float* state,
                     long long slot_stride, const int* seq_of_token, const int* cu_seqlens, const int* slots, int n_seqs,
                     int keep, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(H >= 1, "dyt: rows of %d elements", H);
    TQ_REQUIRE(shift == nullptr || (y == nullptr && rows == nullptr && state != nullptr && seq_of_token != nullptr &&
                                    cu_seqlens != nullptr && slots != nullptr),
               "dyt: the shift wants whole steps, the sequences' kept rows and no sum on the way");
    if (y == nullptr) y_dtype = TQ_F32;
    // an element a thread: two tanhf each with the shift, and steps of a few rows still fill the GPU
    const int threads = H >= 1024 ? 256 : 128;
    const int per_thread = R >= 256 ? 4 : 1;                  // long steps have blocks enough
    dim3 grid(R, (H + per_thread * threads - 1) / (per_thread * threads));
    TQ_REQUIRE(grid.y <= 65535, "dyt: rows of %d elements exceed the grid limit", H);
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = H % 4 == 0 && aligned(x) && aligned(y) && aligned(w) && aligned(b) && aligned(out) && aligned(shift) &&
                     aligned(state) && slot_stride % 4 == 0;
    if (vec) {
        dim3 vgrid(R, (H / 4 + threads - 1) / threads);
        TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
            (tq_launch(vgrid, threads, 0, stream)(dyt_vec_kernel<TY, TW, TO>, x, (const TY*)y, scale, rows, alpha, (const TW*)w, (const TW*)b,
                (TO*)out, H, (const TW*)shift, state, slot_stride, seq_of_token, cu_seqlens, slots, keep)))));
    } else {
        TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
            (tq_launch(grid, threads, 0, stream)(dyt_kernel<TY, TW, TO>, x, (const TY*)y, scale, rows, alpha, (const TW*)w, (const TW*)b,
                (TO*)out, H, (const TW*)shift, state, slot_stride, seq_of_token, cu_seqlens, slots, keep)))));
    }
    TQ_CHECK_LAUNCH("dyt");
    if (shift != nullptr && !keep) {
        TQ_DISPATCH(w_dtype, TW,
            (tq_launch(dim3(n_seqs, grid.y), threads, 0, stream)(dyt_keep_last_kernel<TW>, (const float*)x, alpha, (const TW*)w, (const TW*)b, H,
                state, slot_stride, cu_seqlens, slots)));
        TQ_CHECK_LAUNCH("dyt_keep_last");
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// A weighted sum over the depth of a model: hist holds the stream as every layer so far left it, [n][N] fp32.
// Entry `at` is written first as x + scale * (f + bias) (f: a sub-layer's output still to be added, rows of H
// elements; bias [H]; both may be null), then out = sum over j <= at of weights[j] * hist[j].  x and out may be
// the same tensor.
// ---------------------------------------------------------------------------------------
template <typename TY, typename TW>
__global__ void depth_mix_kernel(float* hist, int at, size_t N, const float* x, const TY* __restrict__ f,
                                 const TW* __restrict__ bias, int H, float scale, const float* __restrict__ weights, float* out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < N; i += stride) {
        float v = x[i];
        if (f != nullptr) v += scale * (tq_to_float(f[i]) + (bias ? tq_to_float(bias[i % H]) : 0.f));
        hist[(size_t)at * N + i] = v;
        float acc = weights[at] * v;
        for (int j = at - 1; j >= 0; --j) acc += weights[j] * hist[(size_t)j * N + i];
        out[i] = acc;
    }
}

TQ_EXPORT int tq_depth_mix(float* hist, int at, long long N, const float* x, const void* f, int f_dtype, const void* bias,
                           int bias_dtype, int H, float scale, const float* weights, float* out, cudaStream_t stream) {
    if (N == 0) return 0;
    TQ_REQUIRE(at >= 0 && H >= 1 && N % H == 0, "depth_mix: entry %d, rows of %d in %lld elements", at, H, N);
    if (f == nullptr) f_dtype = TQ_F32;
    if (bias == nullptr) bias_dtype = TQ_F32;
    const int threads = 256;
    long long blocks = (N + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    TQ_DISPATCH(f_dtype, TY, TQ_DISPATCH(bias_dtype, TW,
        (tq_launch((int)blocks, threads, 0, stream)(depth_mix_kernel<TY, TW>, hist, at, (size_t)N, x, (const TY*)f, (const TW*)bias, H,
            scale, weights, out))));
    TQ_CHECK_LAUNCH("depth_mix");
    return 0;
}

// ---------------------------------------------------------------------------------------
// out[t, i] = act(in[t, i] + bias[i]) for fp32 rows: a projection's bias and the activation behind it in one pass
// (act as in tq_map: 0 identity, 1 the square of relu).
// ---------------------------------------------------------------------------------------
template <typename TW, typename TO>
__global__ void bias_map_kernel(const float* __restrict__ in, const TW* __restrict__ bias, TO* __restrict__ out, size_t n, int N, int act) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float v = in[i] + tq_to_float(bias[i % N]);
        if (act == 1) { v = fmaxf(v, 0.f); v = v * v; }
        out[i] = tq_from_float<TO>(v);
    }
}

TQ_EXPORT int tq_bias_map(const float* in, const void* bias, int bias_dtype, void* out, int out_dtype, int T_, int N, int act,
                          cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(N >= 1 && (act == 0 || act == 1), "bias_map: rows of %d, function %d", N, act);
    const long long n = (long long)T_ * N;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    TQ_DISPATCH(bias_dtype, TW, TQ_DISPATCH(out_dtype, TO,
        (tq_launch((int)blocks, threads, 0, stream)(bias_map_kernel<TW, TO>, in, (const TW*)bias, (TO*)out, (size_t)n, N, act))));
    TQ_CHECK_LAUNCH("bias_map");
    return 0;
}
