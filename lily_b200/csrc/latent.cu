// Attention over a low-rank latent of keys and values: what comes before and after the attention kernel itself.
//
// A token's cache row is [latent (rank) | rotated key part (rot)]: one row for all heads, in pages
// [page_size, rank + rot] of a layer [pages, page_size * (rank + rot)].  Per head the unrotated key is W_uk latent
// and the value W_uv latent, so with q' = W_uk^T q_unrotated the score is q' . latent + q_rotated . k_rotated, and
// the head's output is W_uv (sum_j p_j latent_j): the attention kernel runs over the rows as they are cached, all
// heads sharing them, and reads its values out of the first `rank` columns of the key rows.
//
//   latent_prepare  down-projection row -> RMS-normed query latent; RMS-normed key/value latent and the rotated
//                   key part into the token's cache row
//   latent_query    [q' of every head | rotated part of the head's query] -> the queries the attention kernel takes
//   head_gate       per-head outputs times sigmoid(gate of the head) -> the rows the output projection takes
//
// Norms, angles and the sigmoid are float32.
#include "common.cuh"

namespace lily {

// One block per token.  `in` is the token's row of the stacked down-projection (row stride `ld`): the query latent
// at column q0 (q_rank columns), the key/value latent at kv0 (rank columns) followed by the part to rotate (rot
// columns, of which the first rd are rotated in halves and the rest pass).
template <typename T, typename IN>
__global__ void latent_prepare_kernel(const IN* __restrict__ in, int ld, int q0, int q_rank, int kv0, int rank, int rot,
                                      int rd, const float* __restrict__ q_gain, const float* __restrict__ kv_gain,
                                      float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      const int* __restrict__ positions, const int* __restrict__ token_req,
                                      const int* __restrict__ block_table, int bt_stride, T* __restrict__ layer,
                                      int page_size, int write_kv, T* __restrict__ cq) {
    __shared__ float red[33];
    pdl_enter_small();
    const int t = blockIdx.x;
    const IN* row = in + (size_t)t * ld;
    float ssq = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
        const float x = to_float(row[q0 + c]);
        ssq = fmaf(x, x, ssq);
    }
    const float inv_q = rsqrtf(block_sum(ssq, red) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
        cq[(size_t)t * q_rank + c] = from_float<T>((to_float(row[q0 + c]) * inv_q) * q_gain[c]);
    if (!write_kv) return;
    ssq = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float x = to_float(row[kv0 + c]);
        ssq = fmaf(x, x, ssq);
    }
    const float inv_kv = rsqrtf(block_sum(ssq, red) / (float)rank + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)token_req[t] * bt_stride + pos / page_size];
    const int width = rank + rot;
    T* dst = layer + ((size_t)page * page_size + pos % page_size) * width;
    for (int c = threadIdx.x; c < rank; c += blockDim.x)
        dst[c] = from_float<T>((to_float(row[kv0 + c]) * inv_kv) * kv_gain[c]);
    const int half = rd / 2;
    const IN* kr = row + kv0 + rank;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float u = to_float(kr[i]), v = to_float(kr[i + half]);
        const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
        dst[rank + i] = from_float<T>(u * c - v * s);
        dst[rank + i + half] = from_float<T>(v * c + u * s);
    }
    for (int i = rd + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = from_float<T>(to_float(kr[i]));
}

// grid (tokens, heads).  qa [heads, tokens, rank] (T or float32): the heads' unrotated query parts carried into the
// latent's space; q [tokens, heads, d + rot]: the up-projected queries, of which the last rot columns of a head
// are rotated here.  out [tokens, heads, rank + rot].
template <typename T, typename QA>
__global__ void latent_query_kernel(const QA* __restrict__ qa, const T* __restrict__ q, int tokens, int heads, int d,
                                    int rank, int rot, int rd, const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, const int* __restrict__ positions,
                                    T* __restrict__ out) {
    pdl_enter_small();
    const int t = blockIdx.x, h = blockIdx.y;
    const QA* src = qa + ((size_t)h * tokens + t) * rank;
    T* dst = out + ((size_t)t * heads + h) * (rank + rot);
    for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_float<T>(to_float(src[c]));
    const T* qr = q + ((size_t)t * heads + h) * (d + rot) + d;
    const int pos = positions[t], half = rd / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float u = to_float(qr[i]), v = to_float(qr[i + half]);
        const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
        dst[rank + i] = from_float<T>(u * c - v * s);
        dst[rank + i + half] = from_float<T>(v * c + u * s);
    }
    for (int i = rd + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = qr[i];
}

// grid (tokens, heads).  ov [heads, tokens, dv] (T or float32); gate: column g0 + head of the token's row of the
// stacked down-projection (row stride ld).  out [tokens, heads * dv] = ov * sigmoid(gate).
template <typename T, typename OV, typename IN>
__global__ void head_gate_kernel(const OV* __restrict__ ov, const IN* __restrict__ gate, int ld, int g0, int tokens,
                                 int heads, int dv, T* __restrict__ out) {
    pdl_enter_small();
    const int t = blockIdx.x, h = blockIdx.y;
    const float g = 1.f / (1.f + expf(-to_float(gate[(size_t)t * ld + g0 + h])));
    const OV* src = ov + ((size_t)h * tokens + t) * dv;
    T* dst = out + ((size_t)t * heads + h) * dv;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) dst[c] = from_float<T>(to_float(src[c]) * g);
}

}  // namespace lily

using namespace lily;

LILY_API int lily_latent_prepare(const void* in, int in_dtype, int ld, int q0, int q_rank, int kv0, int rank, int rot,
                                 int rd, const float* q_gain, const float* kv_gain, float eps, const float* cos_t,
                                 const float* sin_t, const int* positions, const int* token_req, const int* block_table,
                                 int bt_stride, void* layer, int page_size, int write_kv, void* cq, int tokens, int dtype,
                                 cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(q_rank > 0 && rank > 0 && rot >= 0 && rd >= 0 && rd <= rot && rd % 2 == 0,
                 "latent_prepare: q_rank=%d rank=%d rot=%d rotated=%d", q_rank, rank, rot, rd);
    LILY_REQUIRE(rd == 0 || (cos_t && sin_t), "latent_prepare: rotation needs its tables");
    LILY_REQUIRE(in_dtype == dtype || in_dtype == kF32, "latent_prepare: the input is the activation dtype or float32");
    dim3 grid(tokens), block(128);
#define GO(T, IN)                                                                                                      \
    launch_pdl(latent_prepare_kernel<T, IN>, grid, block, 0, stream, (const IN*)in, ld, q0, q_rank, kv0, rank, rot, rd, \
               q_gain, kv_gain, eps, cos_t, sin_t, positions, token_req, block_table, bt_stride, (T*)layer, page_size,  \
               write_kv, (T*)cq)
    if (dtype == kBF16) {
        if (in_dtype == kF32) GO(__nv_bfloat16, float); else GO(__nv_bfloat16, __nv_bfloat16);
    } else {
        GO(float, float);
    }
#undef GO
    LILY_CHECK_LAUNCH("latent_prepare");
    return 0;
}

LILY_API int lily_latent_query(const void* qa, int qa_dtype, const void* q, int tokens, int heads, int d, int rank, int rot,
                               int rd, const float* cos_t, const float* sin_t, const int* positions, void* out, int dtype,
                               cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(heads > 0 && heads <= 65535 && rank > 0 && rd <= rot && rd % 2 == 0, "latent_query: heads=%d rank=%d rot=%d", heads, rank, rot);
    LILY_REQUIRE(qa_dtype == dtype || qa_dtype == kF32, "latent_query: the input is the activation dtype or float32");
    dim3 grid(tokens, heads), block(128);
#define GO(T, QA)                                                                                                   \
    launch_pdl(latent_query_kernel<T, QA>, grid, block, 0, stream, (const QA*)qa, (const T*)q, tokens, heads, d, rank, \
               rot, rd, cos_t, sin_t, positions, (T*)out)
    if (dtype == kBF16) {
        if (qa_dtype == kF32) GO(__nv_bfloat16, float); else GO(__nv_bfloat16, __nv_bfloat16);
    } else {
        GO(float, float);
    }
#undef GO
    LILY_CHECK_LAUNCH("latent_query");
    return 0;
}

LILY_API int lily_head_gate(const void* ov, int ov_dtype, const void* gate, int gate_dtype, int ld, int g0, int tokens,
                            int heads, int dv, void* out, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(heads > 0 && heads <= 65535 && dv > 0, "head_gate: heads=%d dv=%d", heads, dv);
    LILY_REQUIRE((ov_dtype == dtype || ov_dtype == kF32) && (gate_dtype == dtype || gate_dtype == kF32),
                 "head_gate: inputs are the activation dtype or float32");
    dim3 grid(tokens, heads), block(dv >= 128 ? 128 : (dv >= 64 ? 64 : 32));
#define GO(T, OV, IN)                                                                                              \
    launch_pdl(head_gate_kernel<T, OV, IN>, grid, block, 0, stream, (const OV*)ov, (const IN*)gate, ld, g0, tokens, \
               heads, dv, (T*)out)
    if (dtype == kBF16) {
        const bool of = ov_dtype == kF32, gf = gate_dtype == kF32;
        if (of && gf) GO(__nv_bfloat16, float, float);
        else if (of) GO(__nv_bfloat16, float, __nv_bfloat16);
        else if (gf) GO(__nv_bfloat16, __nv_bfloat16, float);
        else GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    } else {
        GO(float, float, float);
    }
#undef GO
    LILY_CHECK_LAUNCH("head_gate");
    return 0;
}
