// A linear-attention mixer with a decay that depends on the data (the "wkv" recurrence of the RWKV family):
// token shift, the decay's logarithm, and the recurrence itself.
//
// Per request the state lives in one float32 row of a slot table: first the heads' matrices
// [heads, d (key), d (value)], then the mixer's input at the request's last token [width] (the token shift of the
// next step reads it).  A row is zero when its request starts.
//
//   token shift   m_s[t] = h[t] + (h[t - 1] - h[t]) * mu_s            for each of S streams (r, k, v, g, w)
//   decay         lw[t, c] = -exp(w0[c] + sum_j W2[c, j] tanh(a[t, j]))  (the decay's logarithm; decay = exp(lw))
//   recurrence    o_t[j] = sum_i r_t[i] (S[i, j] + u[i] k_t[i] v_t[j]);   S[i, j] <- exp(lw_t[i]) S[i, j] + k_t[i] v_t[j]
//
// Decays, their logarithms, the state and the sums over it are float32 in both precisions.
#include "common.cuh"

namespace lily {

// ---------------------------------------------------------------------------- token shift

// grid (tokens, ceil(width / 256)), block 256: a thread owns one column of one token.  The thread of a request's
// first new token reads the carried input from the slot and is the one that writes the new one (the input at the
// request's last new token), so nothing it reads is written by another thread of the launch.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// VEC = 4: a thread owns four neighbouring columns (width and the state's offset and stride multiples of four, aligned
// bases; the launcher checks); VEC = 1: one column.
template <typename T, int VEC>
__global__ void token_shift_mix_kernel(const T* __restrict__ h, int tokens, int width, const float* __restrict__ mu,
                                       int streams, float* __restrict__ state, size_t state_stride, size_t state_off,
                                       const int* __restrict__ cu_seqlens, const int* __restrict__ token_req,
                                       const int* __restrict__ slots, T* __restrict__ out) {
    pdl_enter_small();
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (c >= width) return;
    const int r = token_req[t];
    const int first = cu_seqlens[r];
    if (VEC == 4) {
        const float4 cur = ld4(h + (size_t)t * width + c);
        float4 prev;
        if (t == first) {
            float* st = state + (size_t)slots[r] * state_stride + state_off + c;
            prev = ld4(st);
            st4(st, ld4(h + (size_t)(cu_seqlens[r + 1] - 1) * width + c));
        } else {
            prev = ld4(h + (size_t)(t - 1) * width + c);
        }
        const float4 diff = make_float4(prev.x - cur.x, prev.y - cur.y, prev.z - cur.z, prev.w - cur.w);
        for (int s = 0; s < streams; ++s) {
            const float4 m = ld4(mu + (size_t)s * width + c);
            st4(out + ((size_t)s * tokens + t) * width + c,
                make_float4(fmaf(diff.x, m.x, cur.x), fmaf(diff.y, m.y, cur.y), fmaf(diff.z, m.z, cur.z), fmaf(diff.w, m.w, cur.w)));
        }
        return;
    }
    const float cur = to_float(h[(size_t)t * width + c]);
    float prev;
    if (t == first) {
        float* st = state + (size_t)slots[r] * state_stride + state_off + c;
        prev = *st;
        *st = to_float(h[(size_t)(cu_seqlens[r + 1] - 1) * width + c]);
    } else {
        prev = to_float(h[(size_t)(t - 1) * width + c]);
    }
    const float diff = prev - cur;
    for (int s = 0; s < streams; ++s)
        out[((size_t)s * tokens + t) * width + c] = from_float<T>(fmaf(diff, mu[(size_t)s * width + c], cur));
}

// ---------------------------------------------------------------------------- the decay's logarithm

// grid (ceil(tokens / 8), ceil(cols / 128)), block 128; a [tokens, rank] float32, w2t [rank, cols] float32 (the second
// matrix of the low-rank pair, transposed so that neighbouring threads read neighbouring numbers), w0 [cols].  A block
// takes eight tokens, so a number of w2t read once serves eight sums.
constexpr int DECAY_TOKENS = 8;
__global__ void wkv_decay_kernel(const float* __restrict__ a, int tokens, int rank, const float* __restrict__ w2t,
                                 const float* __restrict__ w0, int cols, float* __restrict__ lw) {
    extern __shared__ float th[];          // [8][rank]: tanh(a[t, :])
    pdl_enter_small();
    const int t0 = blockIdx.x * DECAY_TOKENS, nt = min(DECAY_TOKENS, tokens - t0);
    for (int i = threadIdx.x; i < DECAY_TOKENS * rank; i += blockDim.x)
        th[i] = i < nt * rank ? tanhf(a[(size_t)t0 * rank + i]) : 0.f;
    __syncthreads();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float z[DECAY_TOKENS];
#pragma unroll
    for (int t = 0; t < DECAY_TOKENS; ++t) z[t] = 0.f;
    for (int j = 0; j < rank; ++j) {
        const float w = w2t[(size_t)j * cols + c];
#pragma unroll
        for (int t = 0; t < DECAY_TOKENS; ++t) z[t] = fmaf(th[t * rank + j], w, z[t]);
    }
    const float b = w0[c];
#pragma unroll
    for (int t = 0; t < DECAY_TOKENS; ++t)
        if (t < nt) lw[(size_t)(t0 + t) * cols + c] = -expf(z[t] + b);
}

// ---------------------------------------------------------------------------- the recurrence

// grid (heads, requests, column blocks), block ceil(d / PC) * ks threads (whole warps, at most 256: wider heads are
// cut by value columns over the third grid axis): `ks` neighbouring lanes share
// PC neighbouring value columns of the head's matrix and hold NPT of its key rows each in registers (rows
// lane * NPT ... of a padded count ks * NPT >= d), so that one r, k and decay read from shared memory serve 2 * PC
// multiply-adds.  The tokens of the request run one after another, staged TT at a time in shared memory.
constexpr int WKV_NPT = 8, WKV_PC = 4, WKV_TT = 16, WKV_PAD = 4;

template <typename T>
__global__ void __launch_bounds__(256, 3) wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, int in_stride,
                                const float* __restrict__ lw, const float* __restrict__ u, float* __restrict__ state,
                                size_t state_stride, float* __restrict__ y, const int* __restrict__ cu_seqlens,
                                const int* __restrict__ slots, int heads, int d, int ks, int mode,
                                const int* __restrict__ item_req, const int* __restrict__ item_start,
                                const int* __restrict__ item_len, float* __restrict__ ws_state,
                                float* __restrict__ ws_decay) {
    extern __shared__ __align__(16) float sm[];
    const int rows = ks * (WKV_NPT + WKV_PAD);              // floats of one token's r (or k, or decay) in shared memory
    float* rs = sm;                                          // [TT][rows]
    float* kk = rs + WKV_TT * rows;
    float* ws = kk + WKV_TT * rows;
    float* vs = ws + WKV_TT * rows;                          // [TT][d]
    float* bonus = vs + WKV_TT * d;                          // [TT]: sum_i r[i] u[i] k[i]
    float* us = bonus + WKV_TT;                              // [d]
    pdl_enter_small();
    // mode 0: blockIdx.y is a request; all its new tokens, from and to the matrices in its slot.
    // modes 1 and 2: blockIdx.y is an item (a chunk of a long portion).  1: from zero, no outputs; leaves the chunk's own
    // matrices and the product of its decays in the workspace.  2: from the matrices the workspace holds for the
    // chunk's start (wkv_combine put them there), writes the outputs and no state.
    const int head = blockIdx.x, item = blockIdx.y;
    // mode 3: as mode 0 for the requests the list names (the short portions of a step that also has long ones).
    const bool whole = mode == 0 || mode == 3;
    const int req = mode == 0 ? item : item_req[item];
    const int tok0 = cu_seqlens[req] + (whole ? 0 : item_start[item]);
    const int n = whole ? cu_seqlens[req + 1] - tok0 : item_len[item];
    if (n <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const int part = tid % ks, col0 = (blockIdx.z * (blockDim.x / ks) + tid / ks) * WKV_PC;  // this thread's key rows and value columns
    const bool live = col0 < d;
    const int hd = heads * d;
    float* st = whole ? state + (size_t)slots[req] * state_stride + (size_t)head * d * d
                          : ws_state + ((size_t)item * heads + head) * d * d;
    float S[WKV_NPT][WKV_PC];
    float wprod[WKV_NPT];                                   // mode 1, first column group: the product of the rows' decays
#pragma unroll
    for (int i = 0; i < WKV_NPT; ++i) wprod[i] = 1.f;
    const bool keeps_decay = mode == 1 && blockIdx.z == 0 && tid / ks == 0;
#pragma unroll
    for (int i = 0; i < WKV_NPT; ++i) {
        const int row = part * WKV_NPT + i;
#pragma unroll
        for (int c = 0; c < WKV_PC; ++c)
            S[i][c] = (mode != 1 && live && row < d && col0 + c < d) ? st[(size_t)row * d + col0 + c] : 0.f;
    }
    for (int i = tid; i < d; i += blockDim.x) us[i] = u[(size_t)head * d + i];
    // rows beyond d read zeros for r and k, so the padded entries of S stay zero and add nothing
    for (int i = tid; i < WKV_TT * rows; i += blockDim.x) { rs[i] = 0.f; kk[i] = 0.f; ws[i] = 0.f; }

    for (int t0 = 0; t0 < n; t0 += WKV_TT) {
        const int tt = min(WKV_TT, n - t0);
        __syncthreads();
        for (int i = tid; i < tt * d; i += blockDim.x) {
            const int t = i / d, c = i - t * d;
            const size_t src = (size_t)(tok0 + t0 + t) * in_stride + (size_t)head * d + c;
            const int at = t * rows + (c / WKV_NPT) * (WKV_NPT + WKV_PAD) + c % WKV_NPT;
            rs[at] = to_float(r[src]);
            kk[at] = to_float(k[src]);
            vs[t * d + c] = to_float(v[src]);
            ws[at] = expf(lw[(size_t)(tok0 + t0 + t) * hd + (size_t)head * d + c]);
        }
        __syncthreads();
        for (int t = warp; t < tt; t += nwarp) {
            float b = 0.f;
            for (int c = lane; c < d; c += 32) {
                const int at = t * rows + (c / WKV_NPT) * (WKV_NPT + WKV_PAD) + c % WKV_NPT;
                b = fmaf(rs[at] * us[c], kk[at], b);
            }
            b = warp_sum(b);
            if (lane == 0) bonus[t] = b;
        }
        __syncthreads();
        for (int t = 0; t < tt; ++t) {
            float vv[WKV_PC], acc[WKV_PC];
#pragma unroll
            for (int c = 0; c < WKV_PC; ++c) {
                vv[c] = (live && col0 + c < d) ? vs[t * d + col0 + c] : 0.f;
                acc[c] = 0.f;
            }
            const float* rp = rs + t * rows + part * (WKV_NPT + WKV_PAD);
            const float* kp = kk + t * rows + part * (WKV_NPT + WKV_PAD);
            const float* wp = ws + t * rows + part * (WKV_NPT + WKV_PAD);
#pragma unroll
            for (int i = 0; i < WKV_NPT; i += 4) {
                const float4 r4 = *reinterpret_cast<const float4*>(rp + i);
                const float4 k4 = *reinterpret_cast<const float4*>(kp + i);
                const float4 w4 = *reinterpret_cast<const float4*>(wp + i);
                const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kq[4] = {k4.x, k4.y, k4.z, k4.w}, wq[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int c = 0; c < WKV_PC; ++c) {
                        if (mode != 1) acc[c] = fmaf(rr[e], S[i + e][c], acc[c]);
                        S[i + e][c] = fmaf(wq[e], S[i + e][c], kq[e] * vv[c]);
                    }
                }
            }
            if (mode != 1) {
#pragma unroll
                for (int c = 0; c < WKV_PC; ++c) {
                    for (int o = 1; o < ks; o <<= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
                }
            }
            if (keeps_decay) {
#pragma unroll
                for (int i = 0; i < WKV_NPT; ++i) wprod[i] *= wp[i];
            }
            if (mode != 1 && live && part == 0) {
                const float bt = bonus[t];
                float* dst = y + (size_t)(tok0 + t0 + t) * hd + (size_t)head * d + col0;
#pragma unroll
                for (int c = 0; c < WKV_PC; ++c)
                    if (col0 + c < d) dst[c] = fmaf(bt, vv[c], acc[c]);
            }
        }
    }
    if (live && mode != 2) {
#pragma unroll
        for (int i = 0; i < WKV_NPT; ++i) {
            const int row = part * WKV_NPT + i;
#pragma unroll
            for (int c = 0; c < WKV_PC; ++c)
                if (row < d && col0 + c < d) st[(size_t)row * d + col0 + c] = S[i][c];
        }
    }
    if (keeps_decay) {
#pragma unroll
        for (int i = 0; i < WKV_NPT; ++i) {
            const int row = part * WKV_NPT + i;
            if (row < d) ws_decay[((size_t)item * heads + head) * d + row] = wprod[i];
        }
    }
}

// Walks the chunks of each long portion in order: S <- diag(decay_c) S + state_c, leaving in the workspace the
// matrices each chunk starts from and in the slot the last ones.  grid (ceil(heads * d * d / 256), long portions).
__global__ void wkv_combine_kernel(float* __restrict__ state, size_t state_stride, const int* __restrict__ slots,
                                   float* __restrict__ ws_state, const float* __restrict__ ws_decay,
                                   const int* __restrict__ long_req, const int* __restrict__ long_first,
                                   const int* __restrict__ long_count, int heads, int d) {
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;               // (head, row, column)
    const int per = heads * d * d;
    if (e >= per) return;
    const int k = blockIdx.y;
    const int head = e / (d * d), row = (e / d) % d;
    float* st = state + (size_t)slots[long_req[k]] * state_stride + e;
    float S = *st;
    const int first = long_first[k], count = long_count[k];
    for (int c0 = 0; c0 < count; c0 += 4) {                             // four chunks' numbers asked for before the first is used
        float local[4], decay[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const bool in = c0 + j < count;
            local[j] = in ? ws_state[(size_t)(first + c0 + j) * per + e] : 0.f;
            decay[j] = in ? ws_decay[((size_t)(first + c0 + j) * heads + head) * d + row] : 1.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (c0 + j < count) {
                ws_state[(size_t)(first + c0 + j) * per + e] = S;
                S = fmaf(decay[j], S, local[j]);
            }
        }
    }
    *st = S;
}


// ---------------------------------------------------------------------------- unit norm by head, gain, gate

// out[t, c] = y[t, c] / rms(y[t, head of c]) * gain[c] * silu(g[t, c]): each group of `gsize` columns is divided by
// its own root mean square; the gate multiplies the normed value.  grid (tokens, ceil(groups / 4)), block 128: a
// warp owns one group of one token.
// VEC = 4: `lanes` neighbouring lanes (a power of two, gsize / 4 of them up to a warp) own a group and hold four
// neighbouring columns a turn, up to four turns, so a warp takes 32 / lanes groups; VEC = 1: a warp a group.
template <typename T, int VEC>
__global__ void group_rmsnorm_gate_kernel(const float* __restrict__ y, const T* __restrict__ g, int g_stride,
                                          const float* __restrict__ gain, T* __restrict__ out, int inner, int gsize,
                                          int groups, float eps, int lanes) {
    pdl_enter_small();
    const size_t t = blockIdx.x;
    const int lane = threadIdx.x & 31;
    if (VEC == 4) {
        const int li = lane % lanes;
        const int grp = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (32 / lanes) + lane / lanes;
        const bool live = grp < groups;
        const int c0 = (live ? grp : 0) * gsize;
        const float* yr = y + t * inner + c0;
        // a group of up to 512 columns stays in the lanes' registers between the two sweeps
        float4 keep[4];
        float ssq = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * (li + lanes * j);
            keep[j] = (live && i < gsize) ? ld4(yr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            ssq += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        if (!live) return;
        const float inv = rsqrtf(ssq / (float)gsize + eps);
        const T* gr = g + t * g_stride + c0;
        T* dst = out + t * inner + c0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * (li + lanes * j);
            if (i < gsize) {
                const float4 z = ld4(gr + i), w = ld4(gain + c0 + i), v = keep[j];
                st4(dst + i, make_float4(((v.x * inv) * w.x) * (z.x / (1.f + expf(-z.x))), ((v.y * inv) * w.y) * (z.y / (1.f + expf(-z.y))),
                                         ((v.z * inv) * w.z) * (z.z / (1.f + expf(-z.z))), ((v.w * inv) * w.w) * (z.w / (1.f + expf(-z.w)))));
            }
        }
        return;
    }
    const int grp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (grp >= groups) return;
    const int c0 = grp * gsize;
    const float* yr = y + t * inner + c0;
    const T* gr = g + t * g_stride + c0;
    T* dst = out + t * inner + c0;
    float ssq = 0.f;
    for (int i = lane; i < gsize; i += 32) ssq = fmaf(yr[i], yr[i], ssq);
    const float inv = rsqrtf(warp_sum(ssq) / (float)gsize + eps);
    for (int i = lane; i < gsize; i += 32) {
        const float z = to_float(gr[i]);
        dst[i] = from_float<T>(((yr[i] * inv) * gain[c0 + i]) * (z / (1.f + expf(-z))));
    }
}

}  // namespace lily

using namespace lily;

LILY_API int lily_token_shift_mix(const void* h, int tokens, int width, const float* mu, int streams, float* state,
                                  size_t state_stride, size_t state_off, const int* cu_seqlens, const int* token_req,
                                  const int* slots, void* out, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(width > 0 && streams > 0, "token_shift_mix: width=%d streams=%d", width, streams);
    const bool vec = width % 4 == 0 && state_off % 4 == 0 && state_stride % 4 == 0 && (uintptr_t)h % 16 == 0 &&
                     (uintptr_t)mu % 16 == 0 && (uintptr_t)state % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int per = vec ? 4 : 1, threads = width / per >= 256 ? 256 : 128;
    dim3 grid(tokens, (width + threads * per - 1) / (threads * per)), block(threads);
    LILY_REQUIRE(grid.y <= 65535, "token_shift_mix: width %d", width);
#define GO(T, V)                                                                                                       \
    launch_pdl(token_shift_mix_kernel<T, V>, grid, block, 0, stream, (const T*)h, tokens, width, mu, streams, state,    \
               state_stride, state_off, cu_seqlens, token_req, slots, (T*)out)
    if (dtype == kBF16) { if (vec) GO(__nv_bfloat16, 4); else GO(__nv_bfloat16, 1); }
    else { if (vec) GO(float, 4); else GO(float, 1); }
#undef GO
    LILY_CHECK_LAUNCH("token_shift_mix");
    return 0;
}

LILY_API int lily_wkv_decay(const float* a, int tokens, int rank, const float* w2t, const float* w0, int cols, float* lw,
                            cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(rank > 0 && cols > 0, "wkv_decay: rank=%d cols=%d", rank, cols);
    dim3 grid((tokens + DECAY_TOKENS - 1) / DECAY_TOKENS, (cols + 127) / 128), block(128);
    LILY_REQUIRE(grid.y <= 65535 && rank <= 1024, "wkv_decay: %d columns, rank %d", cols, rank);
    launch_pdl(wkv_decay_kernel, grid, block, (size_t)DECAY_TOKENS * rank * sizeof(float), stream, a, tokens, rank, w2t, w0, cols, lw);
    LILY_CHECK_LAUNCH("wkv_decay");
    return 0;
}

LILY_API int lily_wkv_max_head_dim() { return 256; }

LILY_API int lily_wkv_scan(const void* r, const void* k, const void* v, int in_stride, const float* lw, const float* u,
                           float* state, size_t state_stride, float* y, const int* cu_seqlens, const int* slots,
                           int requests, int heads, int d, int dtype, int mode, const int* item_req, const int* item_start,
                           const int* item_len, float* ws_state, float* ws_decay, cudaStream_t stream) {
    // requests: the grid's second axis (requests in mode 0, items in modes 1 and 2)
    if (requests == 0) return 0;
    LILY_REQUIRE(mode >= 0 && mode <= 3, "wkv_scan: mode %d", mode);
    LILY_REQUIRE(mode == 0 || item_req, "wkv_scan: a list of requests is needed");
    LILY_REQUIRE(mode == 0 || mode == 3 || (item_start && item_len && ws_state && ws_decay), "wkv_scan: chunks need their lists and a workspace");
    LILY_REQUIRE(heads > 0 && d > 0 && d <= 256, "wkv_scan: %d heads of size %d (sizes up to 256)", heads, d);      // 32 lanes x NPT rows
    LILY_REQUIRE(requests <= 65535, "wkv_scan: %d heads, %d requests", heads, requests);
    int ks = 1;
    while (ks * WKV_NPT < d) ks <<= 1;
    const int groups = (d + WKV_PC - 1) / WKV_PC;                       // groups of PC value columns
    int threads = (groups * ks + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    const int per_block = threads / ks;
    const size_t smem = sizeof(float) * ((size_t)3 * WKV_TT * ks * (WKV_NPT + WKV_PAD) + (size_t)WKV_TT * d + WKV_TT + d);
    dim3 grid(heads, requests, (groups + per_block - 1) / per_block), block(threads);
#define GO(T)                                                                                                         \
    do {                                                                                                              \
        static size_t granted = 48 * 1024;                                                                            \
        if (smem > granted) {                                                                                         \
            cudaError_t e = cudaFuncSetAttribute(wkv_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("wkv_scan: cannot get %zu bytes of shared memory", smem); return 2; }    \
            granted = smem;                                                                                           \
        }                                                                                                             \
        launch_pdl(wkv_scan_kernel<T>, grid, block, smem, stream, (const T*)r, (const T*)k, (const T*)v, in_stride, lw, u, \
                   state, state_stride, y, cu_seqlens, slots, heads, d, ks, mode, item_req, item_start, item_len, ws_state, \
                   ws_decay);                                                                                         \
    } while (0)
    if (dtype == kBF16) GO(__nv_bfloat16); else GO(float);
#undef GO
    LILY_CHECK_LAUNCH("wkv_scan");
    return 0;
}

LILY_API int lily_group_rmsnorm_gate(const float* y, const void* g, int g_stride, const float* gain, void* out, int tokens,
                                     int inner, int groups, float eps, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(groups >= 1 && inner % groups == 0, "group_rmsnorm_gate: %d columns in %d groups", inner, groups);
    const int gsize = inner / groups;
    const size_t item = dtype == kBF16 ? 2 : 4;
    int lanes = 32;                                               // lanes a group in the vector form: gsize / 4, up to a warp
    while (lanes > 1 && lanes * 4 > gsize) lanes >>= 1;
    const bool vec = gsize % 4 == 0 && gsize <= 16 * lanes && g_stride % 4 == 0 &&
                     (uintptr_t)y % 16 == 0 && (uintptr_t)gain % 16 == 0 && (uintptr_t)g % (4 * item) == 0 &&
                     (uintptr_t)out % (4 * item) == 0;
    const int per_block = vec ? 4 * (32 / lanes) : 4;              // groups a block of four warps takes
    dim3 grid(tokens, (groups + per_block - 1) / per_block), block(128);
    LILY_REQUIRE(grid.y <= 65535, "group_rmsnorm_gate: %d groups", groups);
#define GO(T, V)                                                                                                    \
    launch_pdl(group_rmsnorm_gate_kernel<T, V>, grid, block, 0, stream, y, (const T*)g, g_stride, gain, (T*)out, inner, \
               gsize, groups, eps, lanes)
    if (dtype == kBF16) { if (vec) GO(__nv_bfloat16, 4); else GO(__nv_bfloat16, 1); }
    else { if (vec) GO(float, 4); else GO(float, 1); }
#undef GO
    LILY_CHECK_LAUNCH("group_rmsnorm_gate");
    return 0;
}

LILY_API int lily_wkv_combine(float* state, size_t state_stride, const int* slots, float* ws_state, const float* ws_decay,
                              const int* long_req, const int* long_first, const int* long_count, int longs, int heads, int d,
                              cudaStream_t stream) {
    if (longs == 0) return 0;
    const int per = heads * d * d;
    launch_pdl(wkv_combine_kernel, dim3((per + 255) / 256, longs), dim3(256), 0, stream, state, state_stride, slots, ws_state,
               ws_decay, long_req, long_first, long_count, heads, d);
    LILY_CHECK_LAUNCH("wkv_combine");
    return 0;
}
