// Kernels of the state-space mixer (Mamba-2 / state-space duality): the short causal convolution with its
// carried inputs, the selective scan with its carried state, and the gated, grouped RMSNorm behind it.
//
// Everything that enters the recurrence is float32: the step size softplus(dt + bias), the decay
// exp(-exp(A_log) * dt), the state and the sums over it.  Activations (`T`) are float or bfloat16.
//
// Per request the state lives in one float32 row of a slot table: first the scan state
// [heads][head_dim][state] (state index fastest), then the last (taps - 1) inputs of the convolution
// [(taps - 1)][channels], oldest first.  A request's row is zero when it starts.
//
//   conv:  u_t[c] = silu(bias[c] + sum_j w[c][j] * in_(t - (taps-1) + j)[c])        (inputs before the start are 0)
//   scan:  S_t = exp(a * dt_t) S_(t-1) + dt_t * B_t x_t^T,   y_t = S_t^T C_t + D x_t     per head, a = -exp(A_log)
//   norm:  v = y * silu(z);  out = v / sqrt(mean_over_group(v^2) + eps) * gain
#include "common.cuh"

namespace lily {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ---------------------------------------------------------------------------- causal convolution + SiLU

// grid (ceil(channels / 128), chunks), block 128: a thread owns one channel of one chunk of up to `chunk_len`
// consecutive new tokens of one request (chunks start at multiples of chunk_len >= taps - 1 from the portion's
// first token, so only a portion's first chunk reads the carried inputs; the thread of that chunk also writes
// them back, after it has read them, so no other thread touches what it reads).
template <typename T, int TAPS>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int in_stride, int col0, int channels,
                                        const float* __restrict__ w, const float* __restrict__ bias,
                                        float* __restrict__ state, size_t state_stride, size_t state_off,
                                        T* __restrict__ out, const int* __restrict__ chunk_req,
                                        const int* __restrict__ chunk_start, int chunk_len,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
    pdl_enter_small();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int r = chunk_req[blockIdx.y], start = chunk_start[blockIdx.y];
    const int tok0 = cu_seqlens[r], len = cu_seqlens[r + 1] - tok0;
    const int n = min(chunk_len, len - start);
    if (n <= 0) return;
    constexpr int K1 = TAPS - 1;
    float* st = state + (size_t)slots[r] * state_stride + state_off + c;
    const T* src = in + (size_t)tok0 * in_stride + col0 + c;
    float win[K1 > 0 ? K1 : 1];
    if (start == 0) {
#pragma unroll
        for (int j = 0; j < K1; ++j) win[j] = st[(size_t)j * channels];
        if (len > chunk_len) {
#pragma unroll
            for (int j = 0; j < K1; ++j) st[(size_t)j * channels] = to_float(src[(size_t)(len - K1 + j) * in_stride]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < K1; ++j) win[j] = to_float(src[(size_t)(start - K1 + j) * in_stride]);
    }
    float wt[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[j] = w[(size_t)c * TAPS + j];
    const float b = bias ? bias[c] : 0.f;
    T* dst = out + (size_t)(tok0 + start) * channels + c;
    for (int t = 0; t < n; t += 4) {                 // four tokens' inputs asked for before the first is used
        float xs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) xs[u] = t + u < n ? to_float(src[(size_t)(start + t + u) * in_stride]) : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t + u < n) {
                const float x = xs[u];
                float acc = b;
#pragma unroll
                for (int j = 0; j < K1; ++j) acc = fmaf(win[j], wt[j], acc);
                acc = fmaf(x, wt[K1], acc);
#pragma unroll
                for (int j = 0; j + 1 < K1; ++j) win[j] = win[j + 1];
                if (K1 > 0) win[K1 - 1] = x;
                dst[(size_t)(t + u) * channels] = from_float<T>(silu_f(acc));
            }
        }
    }
    if (start == 0 && len <= chunk_len) {
#pragma unroll
        for (int j = 0; j < K1; ++j) st[(size_t)j * channels] = win[j];
    }
}

// ---------------------------------------------------------------------------- selective scan

// grid (heads, requests, ceil(head_dim / pb)), block (pb / PC) * ns threads: `ns` neighbouring lanes share PC
// neighbouring value columns of the head's state and hold a run of NPT of their `n_state` entries each in registers
// (PC * NPT numbers a thread, so that one B and one C entry read from shared memory serve 2 * PC multiply-adds); the tokens of the request run one after another, staged `tt` at a time in shared memory (B and C
// of the head's group, the head's x, step sizes and decays).
//
// A work item (blockIdx.y) is a run of consecutive new tokens of one request.  Without item lists it is a request's
// whole portion, from the state in the request's slot to the state in the request's slot (mode 0).  A long portion
// is cut into chunks that run side by side: mode 1 starts each chunk from zero and leaves the chunk's own state and
// the product of its decays in a workspace (EMIT false: no outputs); a combine kernel then walks the chunks in order,
// S <- decay_c S + state_c, leaving in the workspace the state each chunk starts from and in the slot the last one;
// mode 2 runs each chunk again from that state and writes the outputs.
template <typename T, int NPT, int PC, bool EMIT>
__global__ void __launch_bounds__(256, 2)
ssd_scan_kernel(const T* __restrict__ xbc, int channels, const T* __restrict__ proj, int proj_stride,
                int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                const float* __restrict__ d_skip, float* __restrict__ state, size_t state_stride,
                float* __restrict__ y, const int* __restrict__ cu_seqlens,
                const int* __restrict__ slots, int heads, int pd, int n_state, int groups, int ns,
                int pb, int tt, const int* __restrict__ item_req, const int* __restrict__ item_start,
                const int* __restrict__ item_len, int mode, float* __restrict__ chunk_state,
                float* __restrict__ chunk_decay) {
    extern __shared__ __align__(16) float smem[];
    pdl_enter_small();
    // Lane j of the ns lanes that share PC columns holds entries [j * NPT, (j + 1) * NPT) of each column's state.  In
    // shared memory a token's B (and C) is laid out lane by lane in rows of NPT + 4, so that the lanes' 16-byte reads
    // fall into different banks; entries past n_state are zero there and leave their (zero) state entries alone.
    constexpr int ROW = NPT + 4;
    const int h = blockIdx.x, item = blockIdx.y, p0 = blockIdx.z * pb;
    const int r = item_req ? item_req[item] : item;
    const int tid = threadIdx.x, j = tid % ns, pl = (tid / ns) * PC, p = p0 + pl;     // this thread's first column
    const int tok0 = cu_seqlens[r] + (item_start ? item_start[item] : 0);
    const int len = item_len ? item_len[item] : cu_seqlens[r + 1] - cu_seqlens[r];
    if (len <= 0) return;
    const int padded = ns * NPT, row = ns * ROW;
    float* Bs = smem;                        // [tt][ns][ROW]
    float* Cs = Bs + (size_t)tt * row;       // [tt][ns][ROW]
    float* xs = Cs + (size_t)tt * row;       // [tt][pb]
    float* dts = xs + (size_t)tt * pb;       // [tt]
    float* das = dts + tt;                   // [tt]
    const int inner = heads * pd;
    const int g = h / (heads / groups);
    const int bcol = inner + g * n_state, ccol = inner + (groups + g) * n_state;
    float* st = (mode == 0 ? state + (size_t)slots[r] * state_stride : chunk_state + (size_t)item * heads * pd * n_state) +
                (size_t)h * pd * n_state;
    float S[PC][NPT];
#pragma unroll
    for (int c = 0; c < PC; ++c) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = j * NPT + i;
            S[c][i] = (mode != 1 && p + c < pd && n < n_state) ? st[(size_t)(p + c) * n_state + n] : 0.f;
        }
    }
    const float A = -expf(a_log[h]), bias = dt_bias[h], D = d_skip[h];
    float decayed = 1.f;                     // the product of the item's decays
    for (int t0 = 0; t0 < len; t0 += tt) {
        const int now = min(tt, len - t0);
        __syncthreads();
#pragma unroll 4
        for (int ti = 0; ti < now; ++ti) {
            const T* src = xbc + (size_t)(tok0 + t0 + ti) * channels;
            for (int n = tid; n < padded; n += blockDim.x) {
                const int at = ti * row + (n / NPT) * ROW + (n % NPT);
                Bs[at] = n < n_state ? to_float(src[bcol + n]) : 0.f;
                Cs[at] = n < n_state ? to_float(src[ccol + n]) : 0.f;
            }
            for (int q = tid; q < pb; q += blockDim.x)
                xs[ti * pb + q] = p0 + q < pd ? to_float(src[h * pd + p0 + q]) : 0.f;
        }
        if (tid < now) {
            const float dtv = softplus_f(to_float(proj[(size_t)(tok0 + t0 + tid) * proj_stride + dt_col + h]) + bias);
            dts[tid] = dtv;
            das[tid] = expf(A * dtv);
        }
        __syncthreads();
        for (int ti = 0; ti < now; ++ti) {
            const float da = das[ti], dtv = dts[ti];
            decayed *= da;
            const float4* b4 = reinterpret_cast<const float4*>(Bs + ti * row + j * ROW);
            const float4* c4 = reinterpret_cast<const float4*>(Cs + ti * row + j * ROW);
            float xv[PC], coef[PC], acc[PC];
#pragma unroll
            for (int c = 0; c < PC; ++c) {
                xv[c] = xs[ti * pb + pl + c];
                coef[c] = dtv * xv[c];
                acc[c] = 0.f;
            }
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) {
                const float4 bv = b4[q], cv = c4[q];
                const float bb[4] = {bv.x, bv.y, bv.z, bv.w}, cc[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int c = 0; c < PC; ++c) {
                        S[c][4 * q + e] = fmaf(da, S[c][4 * q + e], coef[c] * bb[e]);
                        if (EMIT) acc[c] = fmaf(S[c][4 * q + e], cc[e], acc[c]);
                    }
                }
            }
            if (EMIT) {
#pragma unroll
                for (int c = 0; c < PC; ++c) {
                    for (int o = ns >> 1; o > 0; o >>= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
                    if (j == 0 && p + c < pd) y[(size_t)(tok0 + t0 + ti) * inner + h * pd + p + c] = fmaf(D, xv[c], acc[c]);
                }
            }
        }
    }
    if (mode == 2) return;
#pragma unroll
    for (int c = 0; c < PC; ++c) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = j * NPT + i;
            if (p + c < pd && n < n_state) st[(size_t)(p + c) * n_state + n] = S[c][i];
        }
    }
    if (mode == 1 && tid == 0 && blockIdx.z == 0) chunk_decay[(size_t)item * heads + h] = decayed;
}

// grid (ceil(elements / 256), long portions), block 256: one entry of the scan state through the chunks of a portion.
__global__ void ssd_combine_kernel(float* __restrict__ state, size_t state_stride, const int* __restrict__ slots,
                                   float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                   const int* __restrict__ long_req, const int* __restrict__ long_first,
                                   const int* __restrict__ long_count, int heads, int per_head) {
    pdl_enter_small();
    const size_t elements = (size_t)heads * per_head;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elements) return;
    const int k = blockIdx.y, h = (int)(e / per_head);
    float* st = state + (size_t)slots[long_req[k]] * state_stride + e;
    float S = *st;
    const int first = long_first[k], count = long_count[k];
    for (int c = first; c < first + count; ++c) {
        float* cs = chunk_state + (size_t)c * elements + e;
        const float own = *cs;
        *cs = S;
        S = fmaf(chunk_decay[(size_t)c * heads + h], S, own);
    }
    *st = S;
}

// ---------------------------------------------------------------------------- gate, then grouped RMSNorm

// grid (tokens, groups), block 256: v = y * silu(z) over one group of `gsize` columns, normalised by the
// group's own root mean square, times the gain.
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z, int z_stride,
                                           const float* __restrict__ gain, T* __restrict__ out, int inner,
                                           int gsize, float eps) {
    __shared__ float red[33];
    pdl_enter_small();
    const size_t t = blockIdx.x;
    const int c0 = blockIdx.y * gsize;
    const float* yr = y + t * inner + c0;
    const T* zr = z + t * z_stride + c0;
    float ssq = 0.f;
    // two columns a thread and turn where the group and the rows allow it (even sizes: 8-byte and 4-byte accesses)
    const bool pairs = (gsize & 1) == 0 && (inner & 1) == 0 && (z_stride & 1) == 0 && (c0 & 1) == 0;
    if (pairs) {
        for (int i = 2 * threadIdx.x; i < gsize; i += 2 * blockDim.x) {
            const float2 yv = *reinterpret_cast<const float2*>(yr + i);
            const float v0 = yv.x * silu_f(to_float(zr[i])), v1 = yv.y * silu_f(to_float(zr[i + 1]));
            ssq += v0 * v0 + v1 * v1;
        }
    } else {
        for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
            const float v = yr[i] * silu_f(to_float(zr[i]));
            ssq = fmaf(v, v, ssq);
        }
    }
    const float inv = rsqrtf(block_sum(ssq, red) / (float)gsize + eps);
    T* dst = out + t * inner + c0;
    if (pairs) {
        for (int i = 2 * threadIdx.x; i < gsize; i += 2 * blockDim.x) {
            const float2 yv = *reinterpret_cast<const float2*>(yr + i);
            const float2 gv = *reinterpret_cast<const float2*>(gain + c0 + i);
            const float v0 = yv.x * silu_f(to_float(zr[i])), v1 = yv.y * silu_f(to_float(zr[i + 1]));
            dst[i] = from_float<T>((v0 * inv) * gv.x);
            dst[i + 1] = from_float<T>((v1 * inv) * gv.y);
        }
        return;
    }
    for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
        const float v = yr[i] * silu_f(to_float(zr[i]));
        dst[i] = from_float<T>((v * inv) * gain[c0 + i]);
    }
}

}  // namespace lily

using namespace lily;

LILY_API int lily_conv_max_taps() { return 8; }

LILY_API int lily_causal_conv_silu(const void* in, int in_stride, int col0, int channels, int taps, const float* w,
                                   const float* bias, float* state, size_t state_stride, size_t state_off, void* out,
                                   const int* chunk_req, const int* chunk_start, int chunks, int chunk_len,
                                   const int* cu_seqlens, const int* slots, int dtype, cudaStream_t stream) {
    if (chunks == 0 || channels == 0) return 0;
    LILY_REQUIRE(taps >= 1 && taps <= 8, "causal_conv_silu: %d taps (1 to 8)", taps);
    LILY_REQUIRE(chunk_len >= taps - 1 && chunk_len >= 1, "causal_conv_silu: chunks of %d tokens for %d taps", chunk_len, taps);
    LILY_REQUIRE(chunks <= 65535, "causal_conv_silu: %d chunks", chunks);
    dim3 grid((channels + 127) / 128, chunks), block(128);
#define GO(T, K)                                                                                                     \
    launch_pdl(causal_conv_silu_kernel<T, K>, grid, block, 0, stream, (const T*)in, in_stride, col0, channels, w, bias, \
               state, state_stride, state_off, (T*)out, chunk_req, chunk_start, chunk_len, cu_seqlens, slots)
#define TAPS_CASE(K) case K: if (dtype == kBF16) GO(__nv_bfloat16, K); else GO(float, K); break;
    switch (taps) {
        TAPS_CASE(1) TAPS_CASE(2) TAPS_CASE(3) TAPS_CASE(4) TAPS_CASE(5) TAPS_CASE(6) TAPS_CASE(7) TAPS_CASE(8)
    }
#undef TAPS_CASE
#undef GO
    LILY_CHECK_LAUNCH("causal_conv_silu");
    return 0;
}

LILY_API int lily_ssd_scan_max_state() { return 512; }

LILY_API int lily_ssd_scan(const void* xbc, int channels, const void* proj, int proj_stride, int dt_col,
                           const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                           size_t state_stride, float* y, const int* cu_seqlens, const int* slots, int requests,
                           int heads, int pd, int n_state, int groups, int dtype, const int* item_req,
                           const int* item_start, const int* item_len, int mode, float* chunk_state, float* chunk_decay,
                           cudaStream_t stream) {
    if (requests == 0) return 0;
    LILY_REQUIRE(mode >= 0 && mode <= 2 && (mode == 0 || (chunk_state && chunk_decay && item_req && item_start && item_len)),
                 "ssd_scan: mode %d needs item lists and a workspace", mode);
    LILY_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0, "ssd_scan: %d heads over %d groups", heads, groups);
    LILY_REQUIRE(n_state >= 1 && n_state <= 512 && pd >= 1, "ssd_scan: state %d (1 to 512), head size %d", n_state, pd);
    LILY_REQUIRE(requests <= 65535, "ssd_scan: %d requests", requests);
    // ns lanes share pc value columns, each lane with npt = 4, 8 or 16 entries of a column's state
    int npt = n_state <= 32 ? 4 : (n_state <= 128 ? 8 : 16);
    int ns = 1;
    while (ns * npt < n_state) ns <<= 1;
    if (ns > 32) { ns = 32; npt = 16; }
    if (npt == 8 && ns >= 16) { npt = 16; ns >>= 1; }    // fewer lanes to add up over
    int pc = pd % 4 == 0 && pd >= 16 ? 4 : (pd % 2 == 0 && pd >= 8 ? 2 : 1);
    const int lanes_cols = 32 / ns > 0 ? 32 / ns : 1;    // column groups that fill a warp
    int groups_needed = (pd + pc - 1) / pc;              // column groups of a head
    int cg = groups_needed;                              // column groups a block: the whole head when it fits 256 threads
    while (cg * ns > 256) cg = (cg + 1) / 2;
    cg = (cg + lanes_cols - 1) / lanes_cols * lanes_cols;    // whole warps
    const int pb = cg * pc;
    const int row = ns * (npt + 4);                      // a token's B (or C) in shared memory, padded lane by lane
    int tt = 16;
    while (tt > 1 && (size_t)tt * (2 * row + pb + 2) * sizeof(float) > 40 * 1024) tt >>= 1;
    // (a block is whole warps, so it has at least as many threads as a stage has tokens)
    const size_t smem = (size_t)tt * (2 * row + pb + 2) * sizeof(float);
    dim3 grid(heads, requests, (pd + pb - 1) / pb), block(cg * ns);
#define GO(T, N, C, E)                                                                                                 \
    launch_pdl(ssd_scan_kernel<T, N, C, E>, grid, block, smem, stream, (const T*)xbc, channels, (const T*)proj, proj_stride, \
               dt_col, dt_bias, a_log, d_skip, state, state_stride, y, cu_seqlens, slots, heads, pd, n_state, groups, ns, \
               pb, tt, item_req, item_start, item_len, mode, chunk_state, chunk_decay)
#define GO_E(T, N, C) do { if (mode == 1) GO(T, N, C, false); else GO(T, N, C, true); } while (0)
#define GO_C(T, N) do { if (pc == 4) GO_E(T, N, 4); else if (pc == 2) GO_E(T, N, 2); else GO_E(T, N, 1); } while (0)
    if (dtype == kBF16) {
        if (npt == 4) GO_C(__nv_bfloat16, 4); else if (npt == 8) GO_C(__nv_bfloat16, 8); else GO_C(__nv_bfloat16, 16);
    } else {
        if (npt == 4) GO_C(float, 4); else if (npt == 8) GO_C(float, 8); else GO_C(float, 16);
    }
#undef GO_C
#undef GO_E
#undef GO
    LILY_CHECK_LAUNCH("ssd_scan");
    return 0;
}

LILY_API int lily_ssd_combine(float* state, size_t state_stride, const int* slots, float* chunk_state,
                              const float* chunk_decay, const int* long_req, const int* long_first,
                              const int* long_count, int portions, int heads, int per_head, cudaStream_t stream) {
    if (portions == 0) return 0;
    LILY_REQUIRE(portions <= 65535, "ssd_combine: %d portions", portions);
    const size_t elements = (size_t)heads * per_head;
    launch_pdl(ssd_combine_kernel, dim3((unsigned)((elements + 255) / 256), portions), dim3(256), 0, stream, state,
               state_stride, slots, chunk_state, chunk_decay, long_req, long_first, long_count, heads, per_head);
    LILY_CHECK_LAUNCH("ssd_combine");
    return 0;
}

LILY_API int lily_gated_group_rmsnorm(const float* y, const void* z, int z_stride, const float* gain, void* out,
                                      int tokens, int inner, int groups, float eps, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(groups >= 1 && inner % groups == 0, "gated_group_rmsnorm: %d columns in %d groups", inner, groups);
    LILY_REQUIRE(groups <= 65535, "gated_group_rmsnorm: %d groups", groups);
    dim3 grid(tokens, groups), block(256);
    if (dtype == kBF16)
        launch_pdl(gated_group_rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, stream, y, (const __nv_bfloat16*)z, z_stride,
                   gain, (__nv_bfloat16*)out, inner, inner / groups, eps);
    else
        launch_pdl(gated_group_rmsnorm_kernel<float>, grid, block, 0, stream, y, (const float*)z, z_stride, gain,
                   (float*)out, inner, inner / groups, eps);
    LILY_CHECK_LAUNCH("gated_group_rmsnorm");
    return 0;
}
