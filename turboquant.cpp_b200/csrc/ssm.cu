// A state-space mixer with a scalar decay per head (the recurrence of Mamba-2) and the short causal convolution
// in front of it.  Per head a with state S [N, vdim] (fp32, one per sequence, carried from step to step):
//   dt   = softplus(dt_raw + dt_bias_a)
//   S   <- exp(-exp(A_log_a) * dt) * S + dt * B x^T
//   y    = S^T C + D_a x
// B and C [N] belong to the head's group (head a uses group a / (heads / groups)).  x, B and C are the output of
// a causal convolution per channel over the projection's xBC part (`taps` taps, the last on the current token,
// zeros before a sequence's start) followed by silu; the last taps-1 inputs of a sequence are part of its state.
// Everything here is fp32: the projection arrives as fp32, decays, step sizes and the state never leave it.
//   conv_silu          the convolution over the step's tokens, reading the kept inputs for a run's first tokens
//   conv_state_update  the kept inputs after the step (a launch of its own: conv_silu reads the old ones)
//   ssm_scan           the recurrence over each sequence's run of new tokens, a warp per four columns of the state
//   gated_group_norm   y * silu(z), RMS norm in equal groups, weight
//   delta_scan         the delta rule with a decay per key channel (its own header below)
#include <type_traits>

#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define SSM_MAX_TAPS 8
#define SSM_MAX_STATE 256

#define CONV_TOKENS 8          // consecutive tokens of a long step per thread: an input is read once, not once per tap

template <typename TW>
__global__ void conv_silu_kernel(const float* __restrict__ proj, int P, int off, const TW* __restrict__ w,
                                 const TW* __restrict__ b, const float* __restrict__ kept, long long slot_stride,
                                 float* __restrict__ out, int T_, int C, int taps, int per_thread, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int n_seqs) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int tb = blockIdx.x * per_thread, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    // win[SSM_MAX_TAPS - 1 - k] is the input k positions back; wr the tap that meets it (0 beyond the taps)
    float win[SSM_MAX_TAPS], wr[SSM_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < SSM_MAX_TAPS; ++k) {
        win[SSM_MAX_TAPS - 1 - k] = 0.f;
        wr[SSM_MAX_TAPS - 1 - k] = k < taps ? tq_to_float(w[(size_t)c * taps + taps - 1 - k]) : 0.f;
    }
    const float bias = b ? tq_to_float(b[c]) : 0.f;
    const int t_end = min(T_, tb + per_thread);
    for (int t = tb; t < t_end; ++t) {
        const int s = TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE);
        const int i = t - cu_seqlens[s];             // place in the sequence's run of new tokens
        if (t == tb || i == 0) {                     // the thread's first token, or a new sequence: the inputs before it
            const float* old = kept + (size_t)slots[s] * slot_stride;      // [taps-1][C]: inputs of the positions just before the run
#pragma unroll
            for (int k = 1; k < SSM_MAX_TAPS; ++k) {
                if (k < taps) {
                    const int src = i - k;
                    win[SSM_MAX_TAPS - 1 - k] = src >= 0 ? proj[(size_t)(t - k) * P + off + c]
                                                         : old[(size_t)(taps - 1 + src) * C + c];
                }
            }
        }
        win[SSM_MAX_TAPS - 1] = proj[(size_t)t * P + off + c];
        float acc = bias;
#pragma unroll
        for (int k = 0; k < SSM_MAX_TAPS; ++k) acc += wr[k] * win[k];
        out[(size_t)t * C + c] = acc / (1.0f + expf(-acc));
#pragma unroll
        for (int k = 0; k < SSM_MAX_TAPS - 1; ++k) win[k] = win[k + 1];
    }
}

__global__ void conv_state_update_kernel(const float* __restrict__ proj, int P, int off, float* __restrict__ kept,
                                         long long slot_stride, int C, int taps, const int* __restrict__ cu_seqlens,
                                         const int* __restrict__ slots) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = cu_seqlens[s], n = cu_seqlens[s + 1] - first;
    float* old = kept + (size_t)slots[s] * slot_stride;
    float v[SSM_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < SSM_MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
            const int idx = j + n - (taps - 1);          // place in the run of the input that is kept at j from now on
            v[j] = idx >= 0 ? proj[(size_t)(first + idx) * P + off + c] : old[(size_t)(j + n) * C + c];
        }
    }
#pragma unroll
    for (int j = 0; j < SSM_MAX_TAPS - 1; ++j)
        if (j < taps - 1) old[(size_t)j * C + c] = v[j];
}

TQ_EXPORT int tq_conv_silu(const float* proj, int P, int off, const void* w, const void* b, int w_dtype, float* kept,
                           long long slot_stride, float* out, int T_, int C, int taps, const int* seq_of_token,
                           const int* cu_seqlens, const int* slots, int n_seqs, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(C >= 1 && taps >= 1 && taps <= SSM_MAX_TAPS, "conv_silu: %d taps (1..%d)", taps, SSM_MAX_TAPS);
    TQ_REQUIRE(off >= 0 && off + C <= P, "conv_silu: channels %d..%d outside the projection's %d", off, off + C, P);
    const int threads = 128;
    const int per_thread = T_ >= 256 ? CONV_TOKENS : 1;        // short steps keep a thread per token and channel
    dim3 grid((T_ + per_thread - 1) / per_thread, (C + threads - 1) / threads);
    TQ_REQUIRE(grid.y <= 65535, "conv_silu: %d channels exceed the grid limit", C);
    TQ_DISPATCH(w_dtype, TW,
        (tq_launch(grid, threads, 0, stream)(conv_silu_kernel<TW>, proj, P, off, (const TW*)w, (const TW*)b,
                                             (const float*)kept, slot_stride, out, T_, C, taps, per_thread, seq_of_token, cu_seqlens, slots, n_seqs)));
    TQ_CHECK_LAUNCH("conv_silu");
    if (taps > 1) {
        dim3 ugrid(n_seqs, (C + threads - 1) / threads);
        tq_launch(ugrid, threads, 0, stream)(conv_state_update_kernel, proj, P, off, kept, slot_stride, C, taps, cu_seqlens, slots);
        TQ_CHECK_LAUNCH("conv_state_update");
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// ssm_scan: grid (sequences, heads, ceil(vdim / SSM_COLS)), SSM_COLS / SSM_CPW warps per block.  A warp owns
// SSM_CPW neighbouring columns of the head's state (kept column by column, [vdim][N], so the lanes' loads and
// stores are neighbours in memory): lane l keeps rows l, l+32, ... (RPL of them) of each column in registers for
// the whole run, so a step reads its B and C values once for the warp's columns and does three float32 operations
// per element of the state (the product B x, the decayed sum, the sum for y).  The sums of y over the lanes are
// not taken step by step: 32 / SSM_CPW steps leave 32 partial sums per lane, which five rounds of exchanges (31
// shuffles) turn into one whole sum per lane, so the chain of dependent shuffles is paid once per group of steps
// and the state's updates run on meanwhile; a whole group is straight-line code.  No barrier between steps.  The
// run is walked in chunks of TC steps whose B, C, x, step sizes and decays lie in shared memory (rows beyond N as
// zeros, so the state's padding rows stay zero and need no test); a chunk's inputs are fetched into registers,
// all loads in flight together, while the chunk before is computed.
// ---------------------------------------------------------------------------------------
#define SSM_COLS 32           // columns of the state per block

// SSM_CPW columns per warp (4 or 2), SSM_COLS / SSM_CPW warps, 32 / SSM_CPW steps whose sums are taken together
// OUT false: the state is walked on and no output written (y is not touched)
template <typename TW, int RPL, int TC, int SSM_CPW, bool OUT>
__global__ void __launch_bounds__(32 * SSM_COLS / SSM_CPW)
ssm_scan_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ proj, int P, int dt_off,
                const TW* __restrict__ dt_bias, const TW* __restrict__ a_log, const TW* __restrict__ d_skip,
                float* __restrict__ state, long long slot_stride, float* __restrict__ y, int heads, int vdim, int N,
                int groups, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                const float* __restrict__ fixed_decay) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    constexpr int SSM_WARPS = SSM_COLS / SSM_CPW, SSM_GROUP = 32 / SSM_CPW;
    extern __shared__ float4 ssm_smem4[];
    float* ssm_smem = reinterpret_cast<float*>(ssm_smem4);
    constexpr int NP = 32 * RPL;             // rows with padding
    constexpr int NT = 32 * SSM_WARPS;
    float* xs = ssm_smem;                    // [TC][SSM_COLS]  (first: 16-byte reads)
    float* Bs = xs + TC * SSM_COLS;          // [TC][NP]
    float* Cs = Bs + TC * NP;                // [TC][NP]
    float* dts = Cs + TC * NP;               // [TC]
    float* dec = dts + TC;                   // [TC]
    const int s = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * SSM_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int vw = v0 + warp * SSM_CPW;      // the warp's first column
    const int g = h / (heads / groups);
    const int inner = heads * vdim;
    const int first = cu_seqlens[s], n = cu_seqlens[s + 1] - first;
    // fixed_decay: the recurrence S <- decay[h] S + B x^T, y = S^T C with a constant decay per head, a step size of
    // one and no skip term (the per-head constants and the raw step sizes are not read)
    const bool fixed = fixed_decay != nullptr;
    const float A = fixed ? 0.f : -expf(tq_to_float(a_log[h])), bias = fixed ? 0.f : tq_to_float(dt_bias[h]);
    const float D = fixed ? 0.f : tq_to_float(d_skip[h]), decay_h = fixed ? fixed_decay[h] : 0.f;
    float* Sg = state + (size_t)slots[s] * slot_stride + ((size_t)h * N) * vdim;
    float S[RPL][SSM_CPW];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
#pragma unroll
        for (int c = 0; c < SSM_CPW; ++c) {
            const int row = lane + 32 * r;
            S[r][c] = (row < N && vw + c < vdim) ? Sg[(size_t)(vw + c) * N + row] : 0.f;
        }
    }
    constexpr int LPT = TC * NP / NT;                    // B and C values per thread and chunk
    constexpr int XPT = TC * SSM_COLS / NT;              // x values per thread and chunk
    float pb[LPT], pc[LPT], px[XPT], praw = 0.f;
    auto fetch = [&](int t0) {
        const int tc = min(TC, n - t0);
#pragma unroll
        for (int i = 0; i < LPT; ++i) {
            const int k = tid + i * NT, tt = k / NP, r = k % NP;
            pb[i] = pc[i] = 0.f;
            if (tt < tc && r < N) {
                const float* row = xbc + (size_t)(first + t0 + tt) * C + inner + (size_t)g * N + r;
                pb[i] = row[0];
                pc[i] = row[(size_t)groups * N];
            }
        }
#pragma unroll
        for (int i = 0; i < XPT; ++i) {
            const int k = tid + i * NT, tt = k / SSM_COLS, vv = v0 + k % SSM_COLS;
            px[i] = (tt < tc && vv < vdim) ? xbc[(size_t)(first + t0 + tt) * C + (size_t)h * vdim + vv] : 0.f;
        }
        if (tid < tc && !fixed) praw = proj[(size_t)(first + t0 + tid) * P + dt_off + h];
    };
    if (n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += TC) {
        const int tc = min(TC, n - t0);
#pragma unroll
        for (int i = 0; i < LPT; ++i) {
            Bs[tid + i * NT] = pb[i];
            Cs[tid + i * NT] = pc[i];
        }
#pragma unroll
        for (int i = 0; i < XPT; ++i) xs[tid + i * NT] = px[i];
        if (tid < tc) {
            const float raw = praw + bias;
            const float dt = fixed ? 1.0f : (raw > 20.f ? raw : log1pf(expf(raw)));
            dts[tid] = dt;
            dec[tid] = fixed ? decay_h : expf(A * dt);
        }
        __syncthreads();
        if (t0 + TC < n) fetch(t0 + TC);
        for (int t8 = 0; t8 < tc; t8 += SSM_GROUP) {
            // SSM_GROUP steps' partial sums of y (this lane's rows) are kept and added up over the lanes together
            float v[SSM_GROUP * SSM_CPW];
            auto steps = [&](auto full) {        // a whole group runs as straight-line code: its loads can go ahead
#pragma unroll
                for (int j = 0; j < SSM_GROUP; ++j) {
                    const int tt = t8 + j;
#pragma unroll
                    for (int c = 0; c < SSM_CPW; ++c) v[j * SSM_CPW + c] = 0.f;
                    if (decltype(full)::value || tt < tc) {          // the same for the whole block
                        float xv[SSM_CPW];
                        if constexpr (SSM_CPW == 4) {
                            const float4 x4 = *reinterpret_cast<const float4*>(xs + tt * SSM_COLS + warp * SSM_CPW);
                            xv[0] = x4.x; xv[1] = x4.y; xv[2] = x4.z; xv[3] = x4.w;
                        } else {
                            const float2 x2 = *reinterpret_cast<const float2*>(xs + tt * SSM_COLS + warp * SSM_CPW);
                            xv[0] = x2.x; xv[1] = x2.y;
                        }
                        const float a = dec[tt], dt = dts[tt];
#pragma unroll
                        for (int r = 0; r < RPL; ++r) {
                            const float bv = Bs[tt * NP + lane + 32 * r] * dt, cv = Cs[tt * NP + lane + 32 * r];
#pragma unroll
                            for (int c = 0; c < SSM_CPW; ++c) {
                                S[r][c] = a * S[r][c] + bv * xv[c];
                                if constexpr (OUT) v[j * SSM_CPW + c] += S[r][c] * cv;
                            }
                        }
                    }
                }
            };
            if (t8 + SSM_GROUP <= tc) steps(std::true_type{});
            else steps(std::false_type{});
            if constexpr (!OUT) continue;
            // 32 sums over 32 lanes: every round a lane keeps the half of its values that its bit names and gets
            // the other lane's share of that half, so after five rounds lane l holds the whole sum number l
#pragma unroll
            for (int half = 16; half >= 1; half >>= 1) {
                const bool up = lane & half;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float keep = up ? v[i + half] : v[i], send = up ? v[i] : v[i + half];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
                }
            }
            const int tt = t8 + lane / SSM_CPW, c = lane % SSM_CPW;   // SSM_GROUP * SSM_CPW == 32
            if (tt < tc && vw + c < vdim)
                y[(size_t)(first + t0 + tt) * inner + (size_t)h * vdim + vw + c] =
                    v[0] + D * xs[tt * SSM_COLS + warp * SSM_CPW + c];
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
#pragma unroll
        for (int c = 0; c < SSM_CPW; ++c) {
            const int row = lane + 32 * r;
            if (row < N && vw + c < vdim) Sg[(size_t)(vw + c) * N + row] = S[r][c];
        }
    }
}

#define SSM_LAUNCH_OUT(RPL_, TC_, CPW_, OUT_)                                                                      \
    TQ_DISPATCH(w_dtype, TW,                                                                                      \
        (tq_launch(grid, 32 * SSM_COLS / CPW_, smem, stream)(ssm_scan_kernel<TW, RPL_, TC_, CPW_, OUT_>, xbc, C, proj, P, dt_off, \
            (const TW*)dt_bias, (const TW*)a_log, (const TW*)d_skip, state, slot_stride, y, heads, vdim, N, groups, \
            cu_seqlens, slots, fixed_decay)))
#define SSM_LAUNCH(RPL_, TC_, CPW_)                                                                               \
    do {                                                                                                          \
        if (y == nullptr) SSM_LAUNCH_OUT(RPL_, TC_, CPW_, false);                                                 \
        else SSM_LAUNCH_OUT(RPL_, TC_, CPW_, true);                                                               \
    } while (0)

// TQ_SSM_CPW=2: sixteen warps of two columns instead of eight of four (measured slower at every size tried)
static int ssm_cpw() {
    static const int v = [] { const char* e = getenv("TQ_SSM_CPW"); return e && e[0] == '2' ? 2 : 4; }();
    return v;
}

// Warps a launch makes (a warp owns SSM_CPW columns of a head's state): callers that may cut long runs into chunks
// weigh them against the warps the GPU holds.
TQ_EXPORT int tq_ssm_scan_warps(int n_seqs, int heads, int vdim) {
    return n_seqs * heads * ((vdim + SSM_COLS - 1) / SSM_COLS) * (SSM_COLS / ssm_cpw());
}

TQ_EXPORT int tq_ssm_scan(const float* xbc, int C, const float* proj, int P, int dt_off, const void* dt_bias,
                          const void* a_log, const void* d_skip, int w_dtype, float* state, long long slot_stride,
                          float* y, int n_seqs, int heads, int vdim, int N, int groups, const int* cu_seqlens,
                          const int* slots, const float* fixed_decay, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    if (fixed_decay != nullptr) w_dtype = TQ_F32;        // the per-head tensors are not read
    TQ_REQUIRE(heads >= 1 && vdim >= 1 && groups >= 1 && heads % groups == 0, "ssm_scan: %d heads in %d groups", heads, groups);
    TQ_REQUIRE(N >= 1 && N <= SSM_MAX_STATE, "ssm_scan: state size %d (1..%d)", N, SSM_MAX_STATE);
    TQ_REQUIRE(C == heads * vdim + 2 * groups * N, "ssm_scan: %d channels for %d heads x %d and %d groups x %d", C, heads, vdim, groups, N);
    TQ_REQUIRE(fixed_decay != nullptr || (dt_off >= 0 && dt_off + heads <= P), "ssm_scan: the step sizes lie outside the projection");
    const int RPL = N <= 32 ? 1 : (N <= 64 ? 2 : (N <= 128 ? 4 : 8));
    const int NP = 32 * RPL;
    const int TC = NP <= 64 ? 32 : 16;
    dim3 grid(n_seqs, heads, (vdim + SSM_COLS - 1) / SSM_COLS);
    TQ_REQUIRE(heads <= 65535 && grid.z <= 65535, "ssm_scan: sizes exceed the grid limit");
    const size_t smem = (size_t)(2 * TC * NP + TC * SSM_COLS + 2 * TC) * sizeof(float);
    if (ssm_cpw() == 4) {
        if (RPL == 1) SSM_LAUNCH(1, 32, 4);
        else if (RPL == 2) SSM_LAUNCH(2, 32, 4);
        else if (RPL == 4) SSM_LAUNCH(4, 16, 4);
        else SSM_LAUNCH(8, 16, 4);
    } else {
        if (RPL == 1) SSM_LAUNCH(1, 32, 2);
        else if (RPL == 2) SSM_LAUNCH(2, 32, 2);
        else if (RPL == 4) SSM_LAUNCH(4, 16, 2);
        else SSM_LAUNCH(8, 16, 2);
    }
    TQ_CHECK_LAUNCH("ssm_scan");
    return 0;
}

// ---------------------------------------------------------------------------------------
// out[t, g-th part] = rms(y[t, part] * silu(z[t, part])) * w[part]: the gate first, then the norm of each of the
// `norm_groups` equal parts by its own root mean square.  z is `inner` elements of the projection's row from z_off.
// gate_after: the norm first, then the gate: rms(y[t, part]) * w[part] * silu(z[t, part]).  w may be null (no weight).
// gate_kind 1: sigmoid(z) where silu(z) stands above.
// ---------------------------------------------------------------------------------------
#define GGN_KEEP 8
template <typename TW, typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ proj, int P, int z_off,
                                        const TW* __restrict__ w, TO* __restrict__ out, int inner, int gs, float eps,
                                        int gate_after, int gate_kind) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const size_t t = blockIdx.x;
    const int base = blockIdx.y * gs;
    const float* yr = y + t * inner + base;
    const float* zr = proj + t * P + z_off + base;
    auto silu = [gate_kind](float z) { return (gate_kind ? 1.0f : z) / (1.0f + expf(-z)); };     // or the sigmoid alone
    // a thread's (gated) values stay in registers between the sum of squares and the output (up to GGN_KEEP of them;
    // longer parts compute the rest again)
    float keep[GGN_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < GGN_KEEP; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        keep[k] = 0.f;
        if (i < gs) keep[k] = gate_after ? yr[i] : yr[i] * silu(zr[i]);
        ss += keep[k] * keep[k];
    }
    for (int i = threadIdx.x + GGN_KEEP * blockDim.x; i < gs; i += blockDim.x) {
        const float v = gate_after ? yr[i] : yr[i] * silu(zr[i]);
        ss += v * v;
    }
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int k = 0; k < GGN_KEEP; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < gs) {
            float v = keep[k] * rs * (w ? tq_to_float(w[base + i]) : 1.0f);
            if (gate_after) v *= silu(zr[i]);
            out[t * inner + base + i] = tq_from_float<TO>(v);
        }
    }
    for (int i = threadIdx.x + GGN_KEEP * blockDim.x; i < gs; i += blockDim.x) {
        float v = (gate_after ? yr[i] : yr[i] * silu(zr[i])) * rs * (w ? tq_to_float(w[base + i]) : 1.0f);
        if (gate_after) v *= silu(zr[i]);
        out[t * inner + base + i] = tq_from_float<TO>(v);
    }
}

// The same for short parts (up to 32 * GGN_KEEP elements): a warp per part, four parts a block, no block-wide sums.
template <typename TW, typename TO>
__global__ void __launch_bounds__(128)
gated_group_norm_warp_kernel(const float* __restrict__ y, const float* __restrict__ proj, int P, int z_off,
                             const TW* __restrict__ w, TO* __restrict__ out, int inner, int gs, int n_groups, float eps,
                             int gate_after, int gate_kind) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const size_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, g = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (g >= n_groups) return;
    const int base = g * gs;
    const float* yr = y + t * inner + base;
    const float* zr = proj + t * P + z_off + base;
    auto silu = [gate_kind](float z) { return (gate_kind ? 1.0f : z) / (1.0f + expf(-z)); };     // or the sigmoid alone
    float keep[GGN_KEEP], gate[GGN_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < GGN_KEEP; ++k) {
        const int i = lane + 32 * k;
        keep[k] = 0.f;
        gate[k] = 0.f;
        if (i < gs) {
            gate[k] = silu(zr[i]);
            keep[k] = gate_after ? yr[i] : yr[i] * gate[k];
        }
        ss += keep[k] * keep[k];
    }
    ss = tq_warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int k = 0; k < GGN_KEEP; ++k) {
        const int i = lane + 32 * k;
        if (i < gs) {
            float v = keep[k] * rs * (w ? tq_to_float(w[base + i]) : 1.0f);
            if (gate_after) v *= gate[k];
            out[t * inner + base + i] = tq_from_float<TO>(v);
        }
    }
}

TQ_EXPORT int tq_gated_group_norm(const float* y, const float* proj, int P, int z_off, const void* w, int w_dtype,
                                  void* out, int out_dtype, int T_, int inner, int norm_groups, float eps, int gate_after,
                                  int gate_kind, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(inner >= 1 && norm_groups >= 1 && inner % norm_groups == 0 && norm_groups <= 65535,
               "gated_group_norm: %d elements in %d groups", inner, norm_groups);
    TQ_REQUIRE(z_off >= 0 && z_off + inner <= P, "gated_group_norm: the gate lies outside the projection");
    const int gs = inner / norm_groups;
    dim3 grid(T_, norm_groups);
    const int threads = gs >= 1024 ? 256 : (gs >= 128 ? 128 : (gs >= 64 ? 64 : 32));
    if (w == nullptr) w_dtype = TQ_F32;
    if (gs <= 32 * GGN_KEEP && norm_groups >= 4) {
        TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
            (tq_launch(dim3(T_, (norm_groups + 3) / 4), 128, 0, stream)(gated_group_norm_warp_kernel<TW, TO>, y, proj, P, z_off,
                (const TW*)w, (TO*)out, inner, gs, norm_groups, eps, gate_after, gate_kind))));
        TQ_CHECK_LAUNCH("gated_group_norm");
        return 0;
    }
    TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
        (tq_launch(grid, threads, 0, stream)(gated_group_norm_kernel<TW, TO>, y, proj, P, z_off, (const TW*)w, (TO*)out,
                                             inner, gs, eps, gate_after, gate_kind))));
    TQ_CHECK_LAUNCH("gated_group_norm");
    return 0;
}

// ---------------------------------------------------------------------------------------
// What a retention layer's recurrence reads, from a fused projection (fp32 rows of P floats): per token the row
// [v | k' | q'] with k' = rotate(k) * k_scale and q' = rotate(q) (the first rot_dims elements of each head, pairs of
// neighbours or of halves, angle = position * freq[i] in fp32).  q, k: heads x dk from q_off, k_off; v: heads x dv
// from v_off.  The row is the layout of the recurrence's input with one group per head: x = v, B = k', C = q'.
// Grid (token, groups of four heads of k and q): a warp per head; the blocks of a token share out the copy of v.
// ---------------------------------------------------------------------------------------
#define RET_MAX_DIM 256
__global__ void __launch_bounds__(128)
retention_prepare_kernel(const float* __restrict__ proj, int P, int q_off, int k_off, int v_off, float* __restrict__ out,
                         const float* __restrict__ freq, int rot_dims, int halves, float k_scale,
                         const int* __restrict__ positions, int heads, int dk, int dv) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_head[4][RET_MAX_DIM];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = proj + (size_t)t * P;
    const int C = heads * dv + 2 * heads * dk;
    float* dst = out + (size_t)t * C;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < heads * dv; i += gridDim.y * blockDim.x) dst[i] = row[v_off + i];
    const int item = blockIdx.y * 4 + warp;              // k heads, then q heads
    if (item >= 2 * heads) return;
    const int pos = positions[t];
    const bool is_q = item >= heads;
    const int h = is_q ? item - heads : item;
    const float* src = row + (is_q ? q_off : k_off) + (size_t)h * dk;
    float* sh = s_head[warp];
    for (int e = lane; e < dk; e += 32) sh[e] = src[e];
    __syncwarp();
    float* o = dst + heads * dv + (is_q ? heads * dk : 0) + (size_t)h * dk;
    const float f = is_q ? 1.0f : k_scale;
    for (int e = lane; e < dk; e += 32) o[e] = tq_rotated(sh, e, rot_dims, halves, freq, pos) * f;
}

TQ_EXPORT int tq_retention_prepare(const float* proj, int P, int q_off, int k_off, int v_off, float* out, const float* freq,
                                   int rot_dims, int halves, float k_scale, const int* positions, int T_, int heads,
                                   int dk, int dv, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(heads >= 1 && dk >= 1 && dk <= RET_MAX_DIM && dv >= 1, "retention_prepare: bad sizes %d %d %d", heads, dk, dv);
    TQ_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + heads * dk <= P && k_off + heads * dk <= P && v_off + heads * dv <= P,
               "retention_prepare: the heads lie outside the projection's rows of %d", P);
    TQ_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk && (rot_dims == 0 || freq != nullptr),
               "retention_prepare: %d rotated elements of a head of %d", rot_dims, dk);
    TQ_REQUIRE(heads <= 100000, "retention_prepare: %d heads", heads);
    tq_launch(dim3(T_, (2 * heads + 3) / 4), 128, 0, stream)(retention_prepare_kernel, proj, P, q_off, k_off, v_off, out, freq, rot_dims, halves, k_scale,
                                  positions, heads, dk, dv);
    TQ_CHECK_LAUNCH("retention_prepare");
    return 0;
}

// ---------------------------------------------------------------------------------------
// retention_combine: a long run cut into chunks that were scanned side by side, each from a zero state.  With
// ends[c] the state a chunk reached by itself and len_c its tokens, the state the chunk should have started from is
//   start[c0] = the sequence's kept state;  start[c + 1] = decay_h^len_c * start[c] + ends[c]
// (the recurrence is linear in the state), and the last of these is the sequence's new kept state.  One thread per
// element of a sequence's state walks the sequence's chunks; grid (elements / 256, sequences).  A second scan of the
// chunks from starts[] then gives the outputs.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
retention_combine_kernel(float* __restrict__ state, long long slot_stride, const int* __restrict__ slots,
                         const float* __restrict__ ends, float* __restrict__ starts, const int* __restrict__ seq_chunks,
                         const int* __restrict__ cu_chunks, const float* __restrict__ decay, int per_head, int n_elems) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_elems) return;
    const int s = blockIdx.y;
    const float d = decay[e / per_head];
    float* cell = state + (size_t)slots[s] * slot_stride + e;
    float S = *cell;
    for (int c = seq_chunks[s]; c < seq_chunks[s + 1]; ++c) {
        starts[(size_t)c * n_elems + e] = S;
        S = powf(d, (float)(cu_chunks[c + 1] - cu_chunks[c])) * S + ends[(size_t)c * n_elems + e];
    }
    *cell = S;
}

TQ_EXPORT int tq_retention_combine(float* state, long long slot_stride, const int* slots, const float* ends, float* starts,
                                   const int* seq_chunks, const int* cu_chunks, const float* decay, int n_seqs, int heads,
                                   int per_head, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    TQ_REQUIRE(heads >= 1 && per_head >= 1 && n_seqs <= 65535, "retention_combine: %d heads of %d in %d sequences", heads, per_head, n_seqs);
    const int n_elems = heads * per_head;
    tq_launch(dim3((n_elems + 255) / 256, n_seqs), 256, 0, stream)(retention_combine_kernel, state, slot_stride, slots, ends,
                                                                  starts, seq_chunks, cu_chunks, decay, per_head, n_elems);
    TQ_CHECK_LAUNCH("retention_combine");
    return 0;
}

// ---------------------------------------------------------------------------------------
// retention_step: a decode step of retention in one launch, for steps in which every sequence brings one token
// (token t is sequence t).  Grid (token, head), up to sixteen warps.  From the token's row of the fused projection
// [.. q .. k .. v .. g ..]: q' = rotate(q), k' = rotate(k) * k_scale (as retention_prepare), then over the head's
// state, kept column by column [dv][dk]:  S[c] <- decay_h S[c] + k' v_c,  o_c = S[c] . q'  (a warp per group of columns, lanes
// over the rows), then out = o / sqrt(mean(o^2) + eps) * silu(g) (the unit norm over the head, then the gate).
// All float32; out in the activation dtype.  The state is read and written once.
// ---------------------------------------------------------------------------------------
#define RET_STEP_COLS 4
template <typename TO>
__global__ void __launch_bounds__(512)
retention_step_kernel(const float* __restrict__ proj, int P, int q_off, int k_off, int v_off, int g_off,
                      const float* __restrict__ freq, int rot_dims, int halves, float k_scale,
                      const int* __restrict__ positions, float* __restrict__ state, long long slot_stride,
                      const int* __restrict__ slots, const float* __restrict__ decay, TO* __restrict__ out, int heads,
                      int dk, int dv, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_raw[2][RET_MAX_DIM], s_q[RET_MAX_DIM], s_k[RET_MAX_DIM], scratch[33];
    extern __shared__ float s_o[];     // [dv]
    const int t = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = proj + (size_t)t * P;
    for (int e = tid; e < dk; e += blockDim.x) {
        s_raw[0][e] = row[q_off + (size_t)h * dk + e];
        s_raw[1][e] = row[k_off + (size_t)h * dk + e];
    }
    __syncthreads();
    const int pos = positions[t];
    for (int e = tid; e < dk; e += blockDim.x) {
        s_q[e] = tq_rotated(s_raw[0], e, rot_dims, halves, freq, pos);
        s_k[e] = tq_rotated(s_raw[1], e, rot_dims, halves, freq, pos) * k_scale;
    }
    __syncthreads();
    const float d = decay[h];
    float* S = state + (size_t)slots[t] * slot_stride + (size_t)h * dv * dk;
    const float* vr = row + v_off + (size_t)h * dv;
    // a warp takes RET_STEP_COLS columns at a time, their loads in flight together (a step is one pass over a state
    // that nothing else reads: what it costs is the latency of that pass, not its bytes)
    const int n_warps = blockDim.x >> 5;
    for (int c0 = warp * RET_STEP_COLS; c0 < dv; c0 += n_warps * RET_STEP_COLS) {
        float vc[RET_STEP_COLS], acc[RET_STEP_COLS];
#pragma unroll
        for (int j = 0; j < RET_STEP_COLS; ++j) {
            vc[j] = c0 + j < dv ? vr[c0 + j] : 0.f;
            acc[j] = 0.f;
        }
        // all of the group's state in registers first (up to RET_MAX_DIM / 32 rows a lane and column), then the updates
        float sv[RET_MAX_DIM / 32][RET_STEP_COLS];
#pragma unroll
        for (int i = 0; i < RET_MAX_DIM / 32; ++i) {
            const int r = lane + 32 * i;
#pragma unroll
            for (int j = 0; j < RET_STEP_COLS; ++j) sv[i][j] = (r < dk && c0 + j < dv) ? S[(size_t)(c0 + j) * dk + r] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < RET_MAX_DIM / 32; ++i) {
            const int r = lane + 32 * i;
            if (r < dk) {
                const float kr = s_k[r], qr = s_q[r];
#pragma unroll
                for (int j = 0; j < RET_STEP_COLS; ++j) {
                    const float v = d * sv[i][j] + kr * vc[j];
                    if (c0 + j < dv) S[(size_t)(c0 + j) * dk + r] = v;
                    acc[j] += v * qr;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < RET_STEP_COLS; ++j) acc[j] = tq_warp_sum(acc[j]);
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < RET_STEP_COLS; ++j)
                if (c0 + j < dv) s_o[c0 + j] = acc[j];
        }
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = tid; c < dv; c += blockDim.x) ss += s_o[c] * s_o[c];
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* gr = row + g_off + (size_t)h * dv;
    for (int c = tid; c < dv; c += blockDim.x) {
        const float z = gr[c];
        out[((size_t)t * heads + h) * dv + c] = tq_from_float<TO>(s_o[c] * rs * (z / (1.0f + expf(-z))));
    }
}

TQ_EXPORT int tq_retention_step(const float* proj, int P, int q_off, int k_off, int v_off, int g_off, const float* freq,
                                int rot_dims, int halves, float k_scale, const int* positions, float* state,
                                long long slot_stride, const int* slots, const float* decay, void* out, int out_dtype, int T_,
                                int heads, int dk, int dv, float eps, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(heads >= 1 && heads <= 65535 && dk >= 1 && dk <= RET_MAX_DIM && dv >= 1 && dv <= 8192,
               "retention_step: bad sizes %d %d %d", heads, dk, dv);
    TQ_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && g_off >= 0 && q_off + heads * dk <= P && k_off + heads * dk <= P &&
               v_off + heads * dv <= P && g_off + heads * dv <= P, "retention_step: the heads lie outside the projection's rows of %d", P);
    TQ_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk && (rot_dims == 0 || freq != nullptr),
               "retention_step: %d rotated elements of a head of %d", rot_dims, dk);
    const int groups = (dv + RET_STEP_COLS - 1) / RET_STEP_COLS;                  // a warp a group, up to sixteen
    const int threads = 32 * (groups >= 16 ? 16 : (groups >= 8 ? 8 : (groups >= 4 ? 4 : (groups >= 2 ? 2 : 1))));
    TQ_DISPATCH(out_dtype, TO,
        (tq_launch(dim3(T_, heads), threads, (size_t)dv * sizeof(float), stream)(retention_step_kernel<TO>, proj, P, q_off, k_off, v_off,
            g_off, freq, rot_dims, halves, k_scale, positions, state, slot_stride, slots, decay, (TO*)out, heads, dk, dv, eps)));
    TQ_CHECK_LAUNCH("retention_step");
    return 0;
}


// ---------------------------------------------------------------------------------------
// The delta rule with a decay per key channel.  Per head a with state S [dk, dv] (fp32, one per sequence, carried from
// step to step), for every token of a sequence's run in order:
//   S   <- diag(g) S            g = exp(-exp(A_log_a) * softplus(raw + dt_bias)), one decay per key channel
//   u    = beta * (v - S^T k)   beta = sigmoid(raw beta), k the unit vector of the head's key
//   S   <- S + k u^T
//   o    = S^T q                q the unit vector of the head's query times q_scale; it sees the token's own write
// unit(x) = x / sqrt(sum(x^2) + unit_eps).  q and k (kv_heads x dk, head a reads a / (heads / kv_heads)) and v
// (heads x dv) come from xqkv (fp32 rows, the output of conv_silu); raw beta from a projection's fp32 rows; the raw
// decays from fp32 rows of heads x dk.  Everything is fp32.
// Grid (sequence, head, ceil(dv / 16)), four warps: a warp owns four columns of S (kept column by column, [dv][dk]),
// eight lanes a column, lane `sub` of them the rows sub, sub + 8, ... in registers for the whole run.  The run is
// walked in chunks of `tc` tokens whose unit vectors, decays, values and betas the block prepares in shared memory
// (a warp per token; rows beyond dk as zeros, so the state's padding rows stay zero and need no test).
// ---------------------------------------------------------------------------------------
#define DELTA_COLS 16
template <int RPL>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ xqkv, int C, int q_off, int k_off, int v_off,
                  const float* __restrict__ proj, int P, int b_off, const float* __restrict__ a_raw, int A, int a_off,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ state,
                  long long slot_stride, float* __restrict__ y, int heads, int kv_heads, int dk, int dv, float unit_eps,
                  float q_scale, int tc, const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    constexpr int DKP = RPL * 8;
    extern __shared__ float delta_smem[];
    float* sk = delta_smem;                    // [tc][DKP]
    float* sq = sk + (size_t)tc * DKP;
    float* sg = sq + (size_t)tc * DKP;
    float* sv = sg + (size_t)tc * DKP;         // [tc][DELTA_COLS]
    float* sb = sv + (size_t)tc * DELTA_COLS;  // [tc]
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DELTA_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 7;
    const int lc = warp * 4 + (lane >> 3), col = c0 + lc;
    const bool live = col < dv;
    const int g = h / (heads / kv_heads);
    const int t0 = cu_seqlens[s], n = cu_seqlens[s + 1] - t0;
    float* Sp = state + (size_t)slots[s] * slot_stride + ((size_t)h * dv + (live ? col : 0)) * dk;
    float S[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int row = sub + 8 * r;
        S[r] = live && row < dk ? Sp[row] : 0.f;
    }
    const float rate = expf(a_log[h]);
    for (int base = 0; base < n; base += tc) {
        const int nt = min(tc, n - base);
        for (int i = warp; i < nt; i += 4) {
            const size_t t = (size_t)t0 + base + i;
            const float* kr = xqkv + t * C + k_off + (size_t)g * dk;
            const float* qr = xqkv + t * C + q_off + (size_t)g * dk;
            const float* ar = a_raw + t * A + a_off + (size_t)h * dk;
            float ssk = 0.f, ssq = 0.f;
            for (int e = lane; e < dk; e += 32) { ssk += kr[e] * kr[e]; ssq += qr[e] * qr[e]; }
            const float rk = 1.0f / sqrtf(tq_warp_sum(ssk) + unit_eps);
            const float rq = q_scale / sqrtf(tq_warp_sum(ssq) + unit_eps);
            for (int e = lane; e < DKP; e += 32) {
                float kv = 0.f, qv = 0.f, gv = 0.f;
                if (e < dk) {
                    kv = kr[e] * rk;
                    qv = qr[e] * rq;
                    const float z = ar[e] + dt_bias[(size_t)h * dk + e];
                    const float sp = z > 20.f ? z : log1pf(expf(z));
                    gv = expf(-rate * sp);
                }
                sk[i * DKP + e] = kv; sq[i * DKP + e] = qv; sg[i * DKP + e] = gv;
            }
            if (lane < DELTA_COLS) sv[i * DELTA_COLS + lane] = c0 + lane < dv ? xqkv[t * C + v_off + (size_t)h * dv + c0 + lane] : 0.f;
            if (lane == 0) sb[i] = 1.0f / (1.0f + expf(-proj[t * P + b_off + h]));
        }
        __syncthreads();
        for (int i = 0; i < nt; ++i) {
            const float* ki = sk + i * DKP + sub;
            const float* qi = sq + i * DKP + sub;
            const float* gi = sg + i * DKP + sub;
            float pred = 0.f;
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                S[r] *= gi[8 * r];
                pred += S[r] * ki[8 * r];
            }
            pred += __shfl_xor_sync(0xffffffffu, pred, 1);
            pred += __shfl_xor_sync(0xffffffffu, pred, 2);
            pred += __shfl_xor_sync(0xffffffffu, pred, 4);
            const float u = sb[i] * (sv[i * DELTA_COLS + lc] - pred);
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                S[r] += ki[8 * r] * u;
                o += S[r] * qi[8 * r];
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (sub == 0 && live) y[((size_t)t0 + base + i) * heads * dv + (size_t)h * dv + col] = o;
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int row = sub + 8 * r;
            if (row < dk) Sp[row] = S[r];
        }
    }
}

// xqkv fp32 [T, C]; proj fp32 [T, P] (raw beta of head a at b_off + a); a_raw fp32 [T, A] (raw decays of head a from
// a_off + a * dk); dt_bias fp32 [heads * dk]; a_log fp32 [heads]; state fp32 rows of [heads][dv][dk] at slots[s] *
// slot_stride; y fp32 [T, heads * dv].
TQ_EXPORT int tq_delta_scan(const float* xqkv, int C, int q_off, int k_off, int v_off, const float* proj, int P, int b_off,
                            const float* a_raw, int A, int a_off, const float* dt_bias, const float* a_log, float* state,
                            long long slot_stride, float* y, int n_seqs, int heads, int kv_heads, int dk, int dv,
                            float unit_eps, float q_scale, const int* cu_seqlens, const int* slots, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    TQ_REQUIRE(heads >= 1 && kv_heads >= 1 && heads % kv_heads == 0 && heads <= 65535, "delta_scan: %d heads on %d query/key heads", heads, kv_heads);
    TQ_REQUIRE(dk >= 1 && dk <= SSM_MAX_STATE && dv >= 1, "delta_scan: keys of %d elements (1..%d), values of %d", dk, SSM_MAX_STATE, dv);
    TQ_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + kv_heads * dk <= C && k_off + kv_heads * dk <= C && v_off + heads * dv <= C,
               "delta_scan: queries, keys or values lie outside rows of %d", C);
    TQ_REQUIRE(b_off >= 0 && b_off + heads <= P && a_off >= 0 && a_off + heads * dk <= A, "delta_scan: betas or decays lie outside their rows");
    const int rpl = dk <= 64 ? 8 : (dk <= 128 ? 16 : 32);
    const int tc = rpl <= 16 ? 16 : 8;
    const size_t smem = ((size_t)3 * rpl * 8 + DELTA_COLS + 1) * tc * sizeof(float);
    dim3 grid(n_seqs, heads, (dv + DELTA_COLS - 1) / DELTA_COLS);
    TQ_REQUIRE(grid.z <= 65535, "delta_scan: values of %d elements exceed the grid limit", dv);
#define DELTA_LAUNCH(R)                                                                                                 \
    tq_launch(grid, 128, smem, stream)(delta_scan_kernel<R>, xqkv, C, q_off, k_off, v_off, proj, P, b_off, a_raw, A, a_off, \
        dt_bias, a_log, state, slot_stride, y, heads, kv_heads, dk, dv, unit_eps, q_scale, tc, cu_seqlens, slots)
    if (rpl == 8) DELTA_LAUNCH(8); else if (rpl == 16) DELTA_LAUNCH(16); else DELTA_LAUNCH(32);
#undef DELTA_LAUNCH
    TQ_CHECK_LAUNCH("delta_scan");
    return 0;
}

// ---------------------------------------------------------------------------------------
// The delta rule for runs of many tokens, in two launches.
//   delta_prepare: what the recurrence reads, for all tokens side by side: per token a row of `R` floats
//                  [k: G x dk unit vectors | q: G x dk unit vectors times q_scale | g: H x dk decays | k.q: G | beta: H]
//                  (R rounded up to a multiple of four).  A warp per (token, query/key head) and per (token, head).
//   delta_scan_rows: the recurrence over those rows.  Same grid and ownership of the state as delta_scan; a chunk's
//                  rows come through cp.async into one of two buffers in shared memory while the chunk before is
//                  computed.  Per token both read-outs are taken from the decayed state BEFORE the write,
//                  pred = (gS)^T k and r = (gS)^T q, their two chains of shuffles side by side, and the output is
//                  o = r + (k.q) u: the same sum as (gS + k u^T)^T q, with one round of shuffles on the path from a
//                  token's state to the next token's instead of two.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ xqkv, int C, int q_off, int k_off, const float* __restrict__ proj, int P, int b_off,
                     const float* __restrict__ a_raw, int A, int a_off, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, float* __restrict__ rows, int R, int T_, int heads, int kv_heads, int dk,
                     float unit_eps, float q_scale) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31, item = blockIdx.y * 4 + (threadIdx.x >> 5);
    const size_t t = blockIdx.x;
    if (item >= kv_heads + heads) return;
    float* out = rows + t * R;
    const int g_at = 2 * kv_heads * dk, kq_at = g_at + heads * dk, b_at = kq_at + kv_heads;
    if (item < kv_heads) {
        const float* kr = xqkv + t * C + k_off + (size_t)item * dk;
        const float* qr = xqkv + t * C + q_off + (size_t)item * dk;
        float ssk = 0.f, ssq = 0.f;
        for (int e = lane; e < dk; e += 32) { const float a = kr[e], b = qr[e]; ssk += a * a; ssq += b * b; }
        ssk = tq_warp_sum(ssk); ssq = tq_warp_sum(ssq);
        const float rk = 1.0f / sqrtf(ssk + unit_eps), rq = q_scale / sqrtf(ssq + unit_eps);
        for (int e = lane; e < dk; e += 32) {
            out[(size_t)item * dk + e] = kr[e] * rk;
            out[(size_t)(kv_heads + item) * dk + e] = qr[e] * rq;
        }
        // k.q of the vectors as they are written: summed again from the rounded values the recurrence will read
        float kq = 0.f;
        for (int e = lane; e < dk; e += 32) kq += (kr[e] * rk) * (qr[e] * rq);
        kq = tq_warp_sum(kq);
        if (lane == 0) out[kq_at + item] = kq;
    } else {
        const int h = item - kv_heads;
        const float rate = expf(a_log[h]);
        const float* ar = a_raw + t * A + a_off + (size_t)h * dk;
        for (int e = lane; e < dk; e += 32) {
            const float z = ar[e] + dt_bias[(size_t)h * dk + e];
            const float sp = z > 20.f ? z : log1pf(expf(z));
            out[g_at + (size_t)h * dk + e] = expf(-rate * sp);
        }
        if (lane == 0) out[b_at + h] = 1.0f / (1.0f + expf(-proj[t * P + b_off + h]));
    }
}

__device__ __forceinline__ void delta_copy4(float* smem_dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_copy16(float* smem_dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}

template <int RPL>
__global__ void __launch_bounds__(128)
delta_scan_rows_kernel(const float* __restrict__ rows, int R, const float* __restrict__ xqkv, int C, int v_off,
                       float* __restrict__ state, long long slot_stride, float* __restrict__ y, int heads, int kv_heads,
                       int dk, int dv, int tc, int vec, const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    constexpr int DKP = RPL * 8;
    extern __shared__ __align__(16) float delta_rows_smem[];
    const int per_buf = tc * (3 * DKP + DELTA_COLS + 4);       // k, q, g rows, values, k.q, beta (and two unused) per token
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DELTA_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 7;
    const int lc = warp * 4 + (lane >> 3), col = c0 + lc;
    const bool live = col < dv;
    const int g = h / (heads / kv_heads);
    const int t0 = cu_seqlens[s], n = cu_seqlens[s + 1] - t0;
    const int g_at = 2 * kv_heads * dk, kq_at = g_at + heads * dk, b_at = kq_at + kv_heads;
    for (int i = threadIdx.x; i < 2 * per_buf; i += blockDim.x) delta_rows_smem[i] = 0.f;      // rows beyond dk stay zero
    __syncthreads();
    float* Sp = state + (size_t)slots[s] * slot_stride + ((size_t)h * dv + (live ? col : 0)) * dk;
    float S[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int row = sub + 8 * r;
        S[r] = live && row < dk ? Sp[row] : 0.f;
    }
    auto fetch = [&](int base, int buf) {
        float* b = delta_rows_smem + (size_t)buf * per_buf;
        float* bk = b; float* bq = bk + tc * DKP; float* bg = bq + tc * DKP; float* bv = bg + tc * DKP; float* bs = bv + tc * DELTA_COLS;
        const int nt = min(tc, n - base);
        if (vec) {
            const int q4 = dk >> 2;
            for (int i = threadIdx.x; i < nt * q4; i += blockDim.x) {
                const int tk = i / q4, e = (i - tk * q4) * 4;
                const float* src = rows + ((size_t)t0 + base + tk) * R;
                delta_copy16(bk + tk * DKP + e, src + (size_t)g * dk + e);
                delta_copy16(bq + tk * DKP + e, src + (size_t)(kv_heads + g) * dk + e);
                delta_copy16(bg + tk * DKP + e, src + g_at + (size_t)h * dk + e);
            }
        } else {
            for (int i = threadIdx.x; i < nt * dk; i += blockDim.x) {
                const int tk = i / dk, e = i - tk * dk;
                const float* src = rows + ((size_t)t0 + base + tk) * R;
                delta_copy4(bk + tk * DKP + e, src + (size_t)g * dk + e);
                delta_copy4(bq + tk * DKP + e, src + (size_t)(kv_heads + g) * dk + e);
                delta_copy4(bg + tk * DKP + e, src + g_at + (size_t)h * dk + e);
            }
        }
        for (int i = threadIdx.x; i < nt * (DELTA_COLS + 2); i += blockDim.x) {
            const int tk = i / (DELTA_COLS + 2), e = i - tk * (DELTA_COLS + 2);
            const size_t t = (size_t)t0 + base + tk;
            if (e < DELTA_COLS) {
                if (c0 + e < dv) delta_copy4(bv + tk * DELTA_COLS + e, xqkv + t * C + v_off + (size_t)h * dv + c0 + e);
            } else if (e == DELTA_COLS) {
                delta_copy4(bs + tk * 4, rows + t * R + kq_at + g);
            } else {
                delta_copy4(bs + tk * 4 + 1, rows + t * R + b_at + h);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n > 0) fetch(0, 0);
    int buf = 0;
    for (int base = 0; base < n; base += tc, buf ^= 1) {
        const int nt = min(tc, n - base);
        if (base + tc < n) {
            fetch(base + tc, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* b = delta_rows_smem + (size_t)buf * per_buf;
        const float* bk = b + sub; const float* bq = bk + tc * DKP; const float* bg = bq + tc * DKP;
        const float* bv = b + 3 * tc * DKP; const float* bs = bv + tc * DELTA_COLS;
        for (int i = 0; i < nt; ++i) {
            float kreg[RPL];
            float p0 = 0.f, p1 = 0.f, r0 = 0.f, r1 = 0.f;
#pragma unroll
            for (int r = 0; r < RPL; r += 2) {
                kreg[r] = bk[i * DKP + 8 * r];
                kreg[r + 1] = bk[i * DKP + 8 * (r + 1)];
                S[r] *= bg[i * DKP + 8 * r];
                S[r + 1] *= bg[i * DKP + 8 * (r + 1)];
                p0 += S[r] * kreg[r];
                p1 += S[r + 1] * kreg[r + 1];
                r0 += S[r] * bq[i * DKP + 8 * r];
                r1 += S[r + 1] * bq[i * DKP + 8 * (r + 1)];
            }
            float pred = p0 + p1, rd = r0 + r1;
            pred += __shfl_xor_sync(0xffffffffu, pred, 1);
            rd += __shfl_xor_sync(0xffffffffu, rd, 1);
            pred += __shfl_xor_sync(0xffffffffu, pred, 2);
            rd += __shfl_xor_sync(0xffffffffu, rd, 2);
            pred += __shfl_xor_sync(0xffffffffu, pred, 4);
            rd += __shfl_xor_sync(0xffffffffu, rd, 4);
            const float u = bs[i * 4 + 1] * (bv[i * DELTA_COLS + lc] - pred);
#pragma unroll
            for (int r = 0; r < RPL; ++r) S[r] += kreg[r] * u;
            if (sub == 0 && live) y[((size_t)t0 + base + i) * heads * dv + (size_t)h * dv + col] = rd + bs[i * 4] * u;
        }
        __syncthreads();                 // the buffer is free for the chunk after the next
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int row = sub + 8 * r;
            if (row < dk) Sp[row] = S[r];
        }
    }
}

TQ_EXPORT int tq_delta_rows_width(int heads, int kv_heads, int dk) {
    return (2 * kv_heads * dk + heads * dk + kv_heads + heads + 3) / 4 * 4;
}

// The two launches; `rows` is scratch of T * tq_delta_rows_width() floats.  Arguments as for tq_delta_scan.
TQ_EXPORT int tq_delta_scan_runs(const float* xqkv, int C, int q_off, int k_off, int v_off, const float* proj, int P, int b_off,
                                 const float* a_raw, int A, int a_off, const float* dt_bias, const float* a_log, float* rows,
                                 float* state, long long slot_stride, float* y, int T_, int n_seqs, int heads, int kv_heads,
                                 int dk, int dv, float unit_eps, float q_scale, const int* cu_seqlens, const int* slots,
                                 cudaStream_t stream) {
    if (n_seqs == 0 || T_ == 0) return 0;
    TQ_REQUIRE(heads >= 1 && kv_heads >= 1 && heads % kv_heads == 0 && heads <= 65535, "delta_scan_runs: %d heads on %d query/key heads", heads, kv_heads);
    TQ_REQUIRE(dk >= 1 && dk <= SSM_MAX_STATE && dv >= 1, "delta_scan_runs: keys of %d elements (1..%d), values of %d", dk, SSM_MAX_STATE, dv);
    TQ_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + kv_heads * dk <= C && k_off + kv_heads * dk <= C && v_off + heads * dv <= C,
               "delta_scan_runs: queries, keys or values lie outside rows of %d", C);
    TQ_REQUIRE(b_off >= 0 && b_off + heads <= P && a_off >= 0 && a_off + heads * dk <= A, "delta_scan_runs: betas or decays lie outside their rows");
    TQ_REQUIRE(rows != nullptr, "delta_scan_runs: no scratch for the prepared rows");
    const int R = tq_delta_rows_width(heads, kv_heads, dk);
    tq_launch(dim3(T_, (kv_heads + heads + 3) / 4), 128, 0, stream)(delta_prepare_kernel, xqkv, C, q_off, k_off, proj, P, b_off, a_raw, A,
        a_off, dt_bias, a_log, rows, R, T_, heads, kv_heads, dk, unit_eps, q_scale);
    TQ_CHECK_LAUNCH("delta_prepare");
    const int rpl = dk <= 64 ? 8 : (dk <= 128 ? 16 : 32);
    const int tc = rpl <= 16 ? 16 : 8;
    const size_t smem = (size_t)2 * tc * (3 * rpl * 8 + DELTA_COLS + 4) * sizeof(float);
    const int vec = dk % 4 == 0 && ((uintptr_t)rows & 15) == 0;
    dim3 grid(n_seqs, heads, (dv + DELTA_COLS - 1) / DELTA_COLS);
    TQ_REQUIRE(grid.z <= 65535, "delta_scan_runs: values of %d elements exceed the grid limit", dv);
    // Up to an SM's worth of blocks start on an empty GPU, one an SM: launched while the preparation still runs they are
    // packed four an SM where room is first, and the shared-memory pipe they then share makes the scan 2.3 times as long.
    int n_sms = 0, device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
    const bool few_blocks = (long long)grid.x * grid.y * grid.z <= 2LL * n_sms;
#define DELTA_ROWS_LAUNCH(RP)                                                                                          \
    do {                                                                                                               \
        static bool roomy = false;             /* asked for once: two chunks' rows can pass the 48 KB a kernel gets unasked */ \
        if (smem > 48 * 1024 && !roomy) {                                                                              \
            cudaFuncSetAttribute(delta_scan_rows_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);    \
            roomy = true;                                                                                              \
        }                                                                                                              \
        tq_launch(grid, 128, smem, stream, 1, few_blocks ? false : true)(delta_scan_rows_kernel<RP>, (const float*)rows, R, xqkv, C, v_off, state, slot_stride, y, \
            heads, kv_heads, dk, dv, tc, vec, cu_seqlens, slots);                                                      \
    } while (0)
    if (rpl == 8) DELTA_ROWS_LAUNCH(8); else if (rpl == 16) DELTA_ROWS_LAUNCH(16); else DELTA_ROWS_LAUNCH(32);
#undef DELTA_ROWS_LAUNCH
    TQ_CHECK_LAUNCH("delta_scan_rows");
    return 0;
}
