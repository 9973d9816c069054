// A routed mixture of small feed-forward layers: router, grouping of the (token, choice) pairs by expert, the two
// grouped products, and the weighted sum.  Everything stays on the device (no count is read by the host), so a step
// can be captured in a CUDA graph.
//
//   route     z = W_router h (float32); s = softmax(z) over all router outputs; the `top` largest s + correction are
//             chosen; their weights are s / (sum of the chosen s + 1e-20)
//   align     pairs (token, choice) whose expert has weights are grouped by expert: offsets, the pairs in grouped
//             order, each pair's place there, and the list of (expert, first row) tiles the products run over
//   gate/up   a[row, n] = g sigmoid(alpha g) (u + 1), g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit)
//   down      y[row, :] = W_down a[row, :]                                  (float32)
//   combine   out[t] = sum over the token's choices of weight * (y of the pair, or the token's input itself where the
//             chosen router output is one of the last `identity` ones, which have no weights)
//
// Each output number of the products is summed over k in a fixed order, so a pair's result does not depend on what
// else is in the batch.  Router, softmax and the weighted sum are float32.
#include "common.cuh"

namespace lily {

constexpr int ROUTE_MAX = 1024;       // router outputs
constexpr int ROUTE_TOP_MAX = 64;

// grid (ceil(tokens / TB)), block 128: a block takes TB tokens, so a number of the router matrix read once serves TB
// sums (one token a block rereads the matrix from L2 for every token: 50 us for 2,048 tokens of 2,048 columns).
// A token's logits are summed in the same order whatever TB is.
template <typename T, int TB>
__global__ void moe_route_kernel(const T* __restrict__ h, int tokens, int width, const float* __restrict__ router,
                                 const float* __restrict__ correction, int outputs, int top, int* __restrict__ chosen,
                                 float* __restrict__ weights) {
    __shared__ float picked[4][ROUTE_TOP_MAX];
    extern __shared__ __align__(16) float dyn[];             // [TB][width] the tokens' rows, then [TB][outputs] their scores
    float* xs = dyn;
    float* sc = dyn + (size_t)TB * width;
    pdl_enter_small();
    const int t0 = blockIdx.x * TB, nt = min(TB, tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    // the tokens' rows into shared memory as float32, 16 bytes a load where the rows allow (a plain loop of single
    // numbers waits for memory a hundred times over)
    const T* src = h + (size_t)t0 * width;
    constexpr int PER = 16 / (int)sizeof(T);
    if (width % PER == 0 && ((uintptr_t)h & 15) == 0) {
        for (int i = threadIdx.x * PER; i < TB * width; i += blockDim.x * PER) {
            float v[PER];
            if (i < nt * width) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
                const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int u = 0; u < PER; ++u) v[u] = to_float(e[u]);
            } else {
#pragma unroll
                for (int u = 0; u < PER; ++u) v[u] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < PER; u += 4) *reinterpret_cast<float4*>(xs + i + u) = make_float4(v[u], v[u + 1], v[u + 2], v[u + 3]);
        }
    } else {
        for (int i = threadIdx.x; i < TB * width; i += blockDim.x) xs[i] = i < nt * width ? to_float(src[i]) : 0.f;
    }
    __syncthreads();
    for (int e = warp; e < outputs; e += nwarp) {
        const float* w = router + (size_t)e * width;
        float z[TB];
#pragma unroll
        for (int j = 0; j < TB; ++j) z[j] = 0.f;
        if ((width & 3) == 0) {
            // four columns a lane and turn, four turns' numbers of the matrix asked for ahead of their sums
            int c = lane * 4;
            for (; c + 3 * 128 < width; c += 4 * 128) {
                float4 wv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) wv[u] = *reinterpret_cast<const float4*>(w + c + u * 128);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
#pragma unroll
                    for (int j = 0; j < TB; ++j) {
                        const float4 x0 = *reinterpret_cast<const float4*>(xs + j * width + c + u * 128);
                        z[j] = fmaf(x0.x, wv[u].x, fmaf(x0.y, wv[u].y, fmaf(x0.z, wv[u].z, fmaf(x0.w, wv[u].w, z[j]))));
                    }
                }
            }
            for (; c < width; c += 128) {
                const float4 w0 = *reinterpret_cast<const float4*>(w + c);
#pragma unroll
                for (int j = 0; j < TB; ++j) {
                    const float4 x0 = *reinterpret_cast<const float4*>(xs + j * width + c);
                    z[j] = fmaf(x0.x, w0.x, fmaf(x0.y, w0.y, fmaf(x0.z, w0.z, fmaf(x0.w, w0.w, z[j]))));
                }
            }
        } else {
            for (int c = lane; c < width; c += 32) {
                const float wv = w[c];
#pragma unroll
                for (int j = 0; j < TB; ++j) z[j] = fmaf(xs[j * width + c], wv, z[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < TB; ++j) {
            const float total = warp_sum(z[j]);
            if (lane == 0) sc[j * outputs + e] = total;
        }
    }
    __syncthreads();
    // softmax and choice: a warp a token
    for (int j = warp; j < nt; j += nwarp) {
        float* s = sc + j * outputs;
        const int t = t0 + j;
        float mx = -INFINITY;
        for (int e = lane; e < outputs; e += 32) mx = fmaxf(mx, s[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < outputs; e += 32) {
            const float p = expf(s[e] - mx);
            s[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.f / sum;
        __syncwarp();
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = outputs;
            for (int e = lane; e < outputs; e += 32) {
                const float p = s[e];
                if (p < 0.f) continue;                                // taken already
                const float c = p * inv + correction[e];
                if (c > best) { best = c; at = e; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (at >= outputs) at = 0;                                // cannot happen while top <= outputs
            const float p = s[at] * inv;
            total += p;
            __syncwarp();
            if (lane == 0) {
                chosen[(size_t)t * top + k] = at;
                picked[warp][k] = p;
                s[at] = -1.f;
            }
            __syncwarp();
        }
        const float norm = 1.f / (total + 1e-20f);
        for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] = picked[warp][k] * norm;
        __syncwarp();
    }
}

// One block of 1024 threads.  chosen [pairs]; experts: router outputs that have weights (the rest are skipped here).
// offsets [experts + 1], order [pairs] (pairs grouped by expert; entries beyond offsets[experts] are unused),
// place [pairs] (where the pair stands in `order`, -1 without weights), tiles: tile_expert / tile_row [max_tiles]
// (first row of the tile in `order`), tile_count [1].
__global__ void moe_align_kernel(const int* __restrict__ chosen, int pairs, int experts, int rows_per_tile,
                                 int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ place,
                                 int* __restrict__ tile_expert, int* __restrict__ tile_row, int* __restrict__ tile_count,
                                 int max_tiles) {
    extern __shared__ int sh[];            // counts [experts], cursor [experts], start [experts + 1]
    int* counts = sh;
    int* cursor = sh + experts;
    int* start = sh + 2 * experts;
    pdl_enter_small();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = run;
            offsets[e] = run;
            for (int r = 0; r < counts[e] && tiles < max_tiles; r += rows_per_tile) {
                tile_expert[tiles] = e;
                tile_row[tiles] = run + r;
                ++tiles;
            }
            run += counts[e];
        }
        start[experts] = run;
        offsets[experts] = run;
        tile_count[0] = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < experts) {
            const int at = start[e] + atomicAdd(&cursor[e], 1);
            order[at] = p;
            place[p] = at;
        } else {
            place[p] = -1;
        }
    }
}

// The grouped products.  grid (ceil(N / BN), max_tiles), block 256: tile `blockIdx.y` of the list holds up to BM rows
// of one expert.  MODE 0: A rows are the tokens of the pairs (pair / top), W = [gate rows | up rows] of the expert,
// the output is the activation in T.  MODE 1: A rows are the rows of `a` in grouped order, the output float32.
constexpr int EBM = 32, EBN = 64, EBK = 16;

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, size_t w_expert, int N, int K,
                const int* __restrict__ offsets, const int* __restrict__ order, int top,
                const int* __restrict__ tile_expert, const int* __restrict__ tile_row, const int* __restrict__ tile_count,
                void* __restrict__ out, float limit, float alpha) {
    __shared__ float As[EBK][EBM + 4];
    __shared__ float Ws[MODE == 0 ? 2 : 1][EBK][EBN + 4];
    __shared__ int arow[EBM];
    pdl_wait();
    if ((int)blockIdx.y >= tile_count[0]) return;
    const int e = tile_expert[blockIdx.y], row0 = tile_row[blockIdx.y];
    const int rows = min(EBM, offsets[e + 1] - row0);
    const int n0 = blockIdx.x * EBN;
    const T* We = W + (size_t)e * w_expert;
    if (threadIdx.x < EBM) {
        const int r = threadIdx.x;
        arow[r] = r < rows ? (MODE == 0 ? order[row0 + r] / top : row0 + r) : -1;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // 4 columns, 2 rows a thread
    float acc[2][4] = {}, acc2[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += EBK) {
        // A tile: 32 rows x 16 k = 512 numbers, two a thread; W tile(s): 64 rows x 16 k = 1024, four a thread
        for (int i = threadIdx.x; i < EBM * EBK; i += 256) {
            const int r = i / EBK, kk = i % EBK, src = arow[r];
            As[kk][r] = (src >= 0 && k0 + kk < K) ? to_float(A[(size_t)src * lda + k0 + kk]) : 0.f;
        }
        for (int i = threadIdx.x; i < EBN * EBK; i += 256) {
            const int r = i / EBK, kk = i % EBK, n = n0 + r;
            const bool ok = n < N && k0 + kk < K;
            Ws[0][kk][r] = ok ? to_float(We[(size_t)n * K + k0 + kk]) : 0.f;
            if (MODE == 0) Ws[1][kk][r] = ok ? to_float(We[(size_t)(N + n) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < EBK; ++kk) {
            float a[2], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = As[kk][ty * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b[j] = Ws[0][kk][tx * 4 + j];
                if (MODE == 0) b2[j] = Ws[1][kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (MODE == 0) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (MODE == 0) {
                const float g = fminf(acc[i][j], limit);
                const float u = fminf(fmaxf(acc2[i][j], -limit), limit);
                ((T*)out)[(size_t)(row0 + r) * N + n] = from_float<T>((g / (1.f + expf(-alpha * g))) * (u + 1.f));
            } else {
                ((float*)out)[(size_t)(row0 + r) * N + n] = acc[i][j];
            }
        }
    }
}

// grid (tokens, ceil(width / 256)), block 256.  y [pairs in grouped order, width] float32; out [tokens, width] float32.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ h, const int* __restrict__ place,
                                   const float* __restrict__ weights, int top, int width, float* __restrict__ out) {
    pdl_wait();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
        const int at = place[(size_t)t * top + k];
        const float w = weights[(size_t)t * top + k];
        const float v = at >= 0 ? y[(size_t)at * width + c] : to_float(h[(size_t)t * width + c]);
        acc = fmaf(w, v, acc);
    }
    out[(size_t)t * width + c] = acc;
}


// For the library's grouped product (bfloat16, many rows): the pairs' input rows in grouped order, and the activation
// over its gate/up result.  grid (pairs), block 128; rows beyond offsets[experts] (pairs without weights) are zeroed
// so that the product reads nothing unwritten.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, int width, const int* __restrict__ offsets, int experts,
                                  const int* __restrict__ order, int top, T* __restrict__ out) {
    pdl_wait();
    const int row = blockIdx.x;
    const bool live = row < offsets[experts];
    const T* src = h + (size_t)(live ? order[row] / top : 0) * width;
    T* dst = out + (size_t)row * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = live ? src[c] : from_float<T>(0.f);
}

// a[row, n] = g sigmoid(alpha g) (u + 1) from gu[row] = [gate (ff) | up (ff)], clamped as above.
template <typename T>
__global__ void moe_activation_kernel(const T* __restrict__ gu, int ff, T* __restrict__ a, float limit, float alpha) {
    pdl_wait();
    const size_t row = blockIdx.x;
    for (int n = threadIdx.x; n < ff; n += blockDim.x) {
        const float g = fminf(to_float(gu[row * 2 * ff + n]), limit);
        const float u = fminf(fmaxf(to_float(gu[row * 2 * ff + ff + n]), -limit), limit);
        a[row * ff + n] = from_float<T>((g / (1.f + expf(-alpha * g))) * (u + 1.f));
    }
}

// out[t] = sum_k weight * (y[place] or h[t]) with y in the activation dtype (the library product's result)
template <typename T>
__global__ void moe_combine_rows_kernel(const T* __restrict__ y, const T* __restrict__ h, const int* __restrict__ place,
                                        const float* __restrict__ weights, int top, int width, float* __restrict__ out) {
    pdl_wait();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
        const int at = place[(size_t)t * top + k];
        const float w = weights[(size_t)t * top + k];
        const float v = to_float(at >= 0 ? y[(size_t)at * width + c] : h[(size_t)t * width + c]);
        acc = fmaf(w, v, acc);
    }
    out[(size_t)t * width + c] = acc;
}

}  // namespace lily

using namespace lily;

LILY_API int lily_moe_route(const void* h, int tokens, int width, const float* router, const float* correction, int outputs,
                            int top, int* chosen, float* weights, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(outputs >= 1 && outputs <= ROUTE_MAX, "moe_route: %d router outputs (up to %d)", outputs, ROUTE_MAX);
    LILY_REQUIRE(top >= 1 && top <= outputs && top <= ROUTE_TOP_MAX, "moe_route: top %d of %d", top, outputs);
    // four tokens a block once there are blocks enough for the device, and while their rows fit the shared memory
    const int tb = (tokens >= 1024 && (size_t)(4 * width + 4 * outputs) * sizeof(float) <= 40 * 1024) ? 4 : 1;
    const size_t smem = (size_t)tb * (width + outputs) * sizeof(float);
    LILY_REQUIRE(width > 0 && smem <= 44 * 1024, "moe_route: rows of %d numbers and %d outputs do not fit a block's shared memory", width, outputs);
    dim3 grid((tokens + tb - 1) / tb), block(128);
#define GO(T, TB)                                                                                                   \
    launch_pdl(moe_route_kernel<T, TB>, grid, block, smem, stream, (const T*)h, tokens, width, router, correction, outputs, \
               top, chosen, weights)
    if (dtype == kBF16) { if (tb == 4) GO(__nv_bfloat16, 4); else GO(__nv_bfloat16, 1); }
    else { if (tb == 4) GO(float, 4); else GO(float, 1); }
#undef GO
    LILY_CHECK_LAUNCH("moe_route");
    return 0;
}

LILY_API int lily_moe_tile_rows() { return EBM; }

LILY_API int lily_moe_align(const int* chosen, int pairs, int experts, int* offsets, int* order, int* place,
                            int* tile_expert, int* tile_row, int* tile_count, int max_tiles, cudaStream_t stream) {
    LILY_REQUIRE(experts >= 0 && experts <= 4000, "moe_align: %d experts", experts);
    LILY_REQUIRE(max_tiles >= (pairs + EBM - 1) / EBM + experts, "moe_align: room for %d tiles is too little", max_tiles);
    launch_pdl(moe_align_kernel, dim3(1), dim3(1024), (size_t)(3 * experts + 1) * sizeof(int), stream, chosen, pairs, experts,
               EBM, offsets, order, place, tile_expert, tile_row, tile_count, max_tiles);
    LILY_CHECK_LAUNCH("moe_align");
    return 0;
}

// mode 0: gate/up with the activation (W [experts, 2 N, K], out [pairs, N] in the activation dtype);
// mode 1: down (W [experts, N, K], out [pairs, N] float32).
LILY_API int lily_moe_gemm(int mode, const void* A, int lda, const void* W, int N, int K, const int* offsets,
                           const int* order, int top, const int* tile_expert, const int* tile_row, const int* tile_count,
                           int max_tiles, void* out, float limit, float alpha, int dtype, cudaStream_t stream) {
    if (max_tiles == 0 || N == 0) return 0;
    LILY_REQUIRE(K > 0 && lda >= K && (mode == 0 || mode == 1), "moe_gemm: mode=%d N=%d K=%d lda=%d", mode, N, K, lda);
    LILY_REQUIRE(max_tiles <= 65535, "moe_gemm: %d tiles", max_tiles);
    dim3 grid((N + EBN - 1) / EBN, max_tiles), block(256);
    const size_t w_expert = (size_t)(mode == 0 ? 2 : 1) * N * K;
#define GO(T, MODE)                                                                                                \
    launch_pdl(moe_gemm_kernel<T, MODE>, grid, block, 0, stream, (const T*)A, lda, (const T*)W, w_expert, N, K, offsets, \
               order, top, tile_expert, tile_row, tile_count, out, limit, alpha)
    if (dtype == kBF16) { if (mode == 0) GO(__nv_bfloat16, 0); else GO(__nv_bfloat16, 1); }
    else { if (mode == 0) GO(float, 0); else GO(float, 1); }
#undef GO
    LILY_CHECK_LAUNCH("moe_gemm");
    return 0;
}

LILY_API int lily_moe_combine(const float* y, const void* h, const int* place, const float* weights, int tokens, int top,
                              int width, float* out, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    dim3 grid(tokens, (width + 255) / 256), block(256);
    if (dtype == kBF16)
        launch_pdl(moe_combine_kernel<__nv_bfloat16>, grid, block, 0, stream, y, (const __nv_bfloat16*)h, place, weights, top,
                   width, out);
    else
        launch_pdl(moe_combine_kernel<float>, grid, block, 0, stream, y, (const float*)h, place, weights, top, width, out);
    LILY_CHECK_LAUNCH("moe_combine");
    return 0;
}

LILY_API int lily_moe_gather(const void* h, int width, const int* offsets, int experts, const int* order, int top, int pairs,
                             void* out, int dtype, cudaStream_t stream) {
    if (pairs == 0) return 0;
    if (dtype == kBF16)
        launch_pdl(moe_gather_kernel<__nv_bfloat16>, dim3(pairs), dim3(128), 0, stream, (const __nv_bfloat16*)h, width, offsets,
                   experts, order, top, (__nv_bfloat16*)out);
    else
        launch_pdl(moe_gather_kernel<float>, dim3(pairs), dim3(128), 0, stream, (const float*)h, width, offsets, experts, order,
                   top, (float*)out);
    LILY_CHECK_LAUNCH("moe_gather");
    return 0;
}

LILY_API int lily_moe_activation(const void* gu, int ff, int rows, void* a, float limit, float alpha, int dtype,
                                 cudaStream_t stream) {
    if (rows == 0) return 0;
    if (dtype == kBF16)
        launch_pdl(moe_activation_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)gu, ff,
                   (__nv_bfloat16*)a, limit, alpha);
    else
        launch_pdl(moe_activation_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)gu, ff, (float*)a, limit, alpha);
    LILY_CHECK_LAUNCH("moe_activation");
    return 0;
}

LILY_API int lily_moe_combine_rows(const void* y, const void* h, const int* place, const float* weights, int tokens, int top,
                                   int width, float* out, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    dim3 grid(tokens, (width + 255) / 256), block(256);
    if (dtype == kBF16)
        launch_pdl(moe_combine_rows_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)y, (const __nv_bfloat16*)h,
                   place, weights, top, width, out);
    else
        launch_pdl(moe_combine_rows_kernel<float>, grid, block, 0, stream, (const float*)y, (const float*)h, place, weights, top,
                   width, out);
    LILY_CHECK_LAUNCH("moe_combine_rows");
    return 0;
}
