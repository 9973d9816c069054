// Attention over a cached latent in bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulation): all query
// heads share one cached row per position, [latent (rank) | rotated key part], and the values are the first `rank`
// columns of the same rows, so a key tile in shared memory serves the scores (over the whole row) and the weighted
// sum (over its first columns).
//
// The query rows of a request are its (token, head) pairs in that order, which is how they lie in memory.  A block
// takes 32 consecutive rows of a tile of `tile_tokens` new tokens (grid: tiles x ceil(tile_tokens * heads / 32) x
// key ranges) and walks the keys its rows can see in tiles of 64, double-buffered: a cached row is one bulk copy
// (cp.async.bulk, completion counted in bytes on an mbarrier of the buffer), issued by the lanes of the first warp.
// Eight warps: warp w
// owns the 16 rows of row tile w / 4 and, of a key tile, the 16 keys w % 4 for the scores and the value columns
// [w % 4] * VT * 8 ... for the weighted sum.  Per key tile the four warps of a row tile exchange row maxima, the
// weights (bfloat16) and row sums through shared memory, so no score is computed twice.
//
// Decode is the same kernel with one new token a request at position seq_len - 1; its keys may be cut into ranges
// whose (max, sum, output) go to scratch in the layout the combine kernel merges
// (lily_attention_combine: [requests, heads, ranges, rank] outputs, then [.., 2]).
//
// Scores, softmax and sums are float32; the weights are rounded to bfloat16 for their product with the values.
// The wait for a tile is bounded: when it runs out the block records it in a status word (lily_latent_attention_status),
// gives the copies it still has in flight a bounded wait and returns.
#include "attention_args.cuh"
#include "common.cuh"

namespace lily {
namespace latent {

constexpr int BN = 64;            // keys per tile
constexpr int ROWS = 32;          // query rows per block
constexpr int THREADS = 256;
constexpr int PSTRIDE = BN + 8;   // bfloat16 per row of the weights' tile

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
constexpr uint32_t SPIN_LIMIT = 1u << 22;     // polls before a wait for a tile gives up (a fraction of a second)
__device__ int g_status = 0;                  // 0 ok; else 1 + the block of the first wait that gave up

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// `bytes` (a multiple of 16) from global to shared memory, both 16-byte aligned; completes on the mbarrier
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    // not volatile: a register operation, which the compiler may move between the (volatile, ordered) fragment loads
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct Args {
    const __nv_bfloat16* q;       // [tokens, heads, row]
    const __nv_bfloat16* cache;   // [pages, page_size, row]
    __nv_bfloat16* out;           // [tokens, heads, rank]
    const int* block_table;
    int bt_stride;
    const int* cu_seqlens;        // prefill
    const int* prefix_lens;       // prefill
    const int* tile_req;          // prefill
    const int* tile_start;        // prefill
    const int* seq_lens;          // decode
    float* part_o;                // decode with ranges
    float* part_ml;
    int splits, heads, row, rank, page_size, window, tile_tokens;
    int rowp;                     // bfloat16 per row of the query and key tiles in shared memory
    float scale;
};

// VT: tiles of 8 value columns a warp owns (4 * VT * 8 >= rank).
template <int VT, bool DECODE>
__global__ void __launch_bounds__(THREADS, 1) latent_attention_kernel(const Args a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int rowp = a.rowp, rowb = rowp * 2;                       // row stride in elements and bytes
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem);    // [ROWS][rowp]
    __nv_bfloat16* k_s = q_s + ROWS * rowp;                         // [2][BN][rowp]
    __nv_bfloat16* p_s = k_s + 2 * BN * rowp;                       // [2 row tiles][16][PSTRIDE]
    float* smax = reinterpret_cast<float*>(p_s + 2 * 16 * PSTRIDE); // [2][4][16]
    float* ssum = smax + 2 * 4 * 16;                                // [2][4][16]
    __shared__ __align__(8) uint64_t kbar[2];                       // a key buffer's copies have landed
    __shared__ int abort_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mt = warp >> 2, wq = warp & 3;
    const int c = lane & 3, r_lo = lane >> 2, r_hi = r_lo + 8;

    int req, tok0, ntok, pos0, kbeg, kend;
    if (DECODE) {
        req = blockIdx.x;
        tok0 = req;
        ntok = 1;
        const int seq = a.seq_lens[req];
        pos0 = seq - 1;
        const int lo = (a.window > 0 && seq > a.window) ? seq - a.window : 0;
        int per = (seq - lo + a.splits - 1) / a.splits;
        per = (per + BN - 1) / BN * BN;
        kbeg = lo + blockIdx.z * per;
        kend = min(seq, kbeg + per);
    } else {
        req = a.tile_req[blockIdx.x];
        const int start = a.tile_start[blockIdx.x];
        const int first = a.cu_seqlens[req], len = a.cu_seqlens[req + 1] - first;
        tok0 = first + start;
        ntok = min(a.tile_tokens, len - start);
        pos0 = a.prefix_lens[req] + start;
        kend = pos0 + ntok;
        kbeg = (a.window > 0 && pos0 + 1 > a.window) ? pos0 + 1 - a.window : 0;
    }
    const int nrows = ntok * a.heads;                               // rows of the whole tile
    const int row0 = blockIdx.y * ROWS;                             // this block's first row of them
    if (row0 >= nrows) return;
    // this block's rows see keys up to the position of its last row's token, from its first row's window on
    const int last_tok = min(nrows - 1, row0 + ROWS - 1) / a.heads, first_tok = row0 / a.heads;
    kend = min(kend, pos0 + last_tok + 1);
    if (!DECODE && a.window > 0) kbeg = max(kbeg, pos0 + first_tok + 1 - a.window);
    kbeg = max(kbeg, 0);

    // ---- zero the padding columns of every tile row once, stage the queries
    const int chunks = a.row / 8;                                   // 16-byte pieces of a row that hold data
    const int chunks_p = rowp / 8;
    for (int i = tid; i < (ROWS + 2 * BN) * (chunks_p - chunks); i += THREADS) {
        const int r = i / (chunks_p - chunks), ch = chunks + i % (chunks_p - chunks);
        *reinterpret_cast<uint4*>(q_s + (size_t)r * rowp + ch * 8) = make_uint4(0, 0, 0, 0);
    }
    for (int i = tid; i < ROWS * chunks; i += THREADS) {
        const int r = i / chunks, ch = i % chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row0 + r < nrows) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)tok0 * a.heads + row0 + r) * a.row + ch * 8);
        *reinterpret_cast<uint4*>(q_s + (size_t)r * rowp + ch * 8) = v;
    }

    const int* table = a.block_table + (size_t)req * a.bt_stride;
    // the first warp's lanes copy whole cached rows, a bulk copy a row; rows past the last key are zeroed by hand
    const uint32_t bar0 = smem_u32(&kbar[0]);
    const uint32_t row_bytes = (uint32_t)a.row * 2;
    auto load_tile = [&](int t, int buf) {
        if (warp != 0) return;
        const int kb = kbeg + t * BN;
        const int valid = min(BN, kend - kb);
        const uint32_t bar = bar0 + 8 * buf;
        __nv_bfloat16* dst = k_s + (size_t)buf * BN * rowp;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)valid * row_bytes);
        __syncwarp();
        for (int j = lane; j < BN; j += 32) {
            if (j < valid) {
                const int kpos = kb + j;
                const __nv_bfloat16* src = a.cache + ((size_t)table[kpos / a.page_size] * a.page_size + kpos % a.page_size) * a.row;
                bulk_copy(smem_u32(dst + (size_t)j * rowp), src, row_bytes, bar);
            } else {
                for (int ch = 0; ch < chunks; ++ch) *reinterpret_cast<uint4*>(dst + (size_t)j * rowp + ch * 8) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    const int ntiles = kend > kbeg ? (kend - kbeg + BN - 1) / BN : 0;
    if (tid == 0) {
        abort_s = 0;
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();                                        // the barriers are set up (and the queries staged)
    if (ntiles > 0) load_tile(0, 0);

    // positions of this thread's two rows (rows beyond the tile see nothing)
    const int gr_lo = row0 + mt * 16 + r_lo, gr_hi = row0 + mt * 16 + r_hi;
    const int qpos_lo = gr_lo < nrows ? pos0 + gr_lo / a.heads : -1, qpos_hi = gr_hi < nrows ? pos0 + gr_hi / a.heads : -1;

    const float sl2 = a.scale * 1.4426950408889634f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[VT][4];
#pragma unroll
    for (int j = 0; j < VT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const int ksteps = (a.row + 15) / 16;
    const unsigned char* qb = reinterpret_cast<const unsigned char*>(q_s) + (size_t)(mt * 16 + (lane & 15)) * rowb + ((lane >> 4) << 4);
    unsigned char* pb = reinterpret_cast<unsigned char*>(p_s + (size_t)mt * 16 * PSTRIDE);
    float* my_max = smax + mt * 64;
    float* my_sum = ssum + mt * 64;

    for (int t = 0; t < ntiles; ++t) {
        const int buf = t & 1;
        {
            // tile t has landed when its buffer's barrier has passed the phase of this use
            const uint32_t bar = bar0 + 8 * buf, parity = (uint32_t)(t >> 1) & 1;
            bool ok = false;
            for (uint32_t i = 0; i < SPIN_LIMIT && !ok; ++i) {
                ok = mbar_try_wait(bar, parity);
                if (!ok && (i & 1023u) == 1023u && *(volatile int*)&abort_s) break;
            }
            if (!ok) {
                abort_s = 1;
                atomicCAS(&g_status, 0, 1 + (int)(blockIdx.x + blockIdx.y * gridDim.x));
            }
        }
        __syncthreads();                                    // everyone has tile t and is done with tile t - 1
        if (*(volatile int*)&abort_s) {
            // a copy of the tile asked for ahead may still be on its way into this block's shared memory
            if (tid == 0)
                for (uint32_t i = 0; i < SPIN_LIMIT && !mbar_try_wait(bar0 + 8 * buf, (uint32_t)(t >> 1) & 1); ++i) {}
            return;
        }
        if (t + 1 < ntiles) load_tile(t + 1, buf ^ 1);
        const unsigned char* kt = reinterpret_cast<const unsigned char*>(k_s + (size_t)buf * BN * rowp);
        const int kb = kbeg + t * BN;

        // ---- this warp's scores: 16 rows x keys [wq * 16, wq * 16 + 16) of the tile
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        const unsigned char* kr = kt + (size_t)(wq * 16 + (lane & 7) + ((lane >> 4) << 3)) * rowb + (((lane >> 3) & 1) << 4);
        {
            // the fragments of the next step are asked for before this step's products are issued; even and odd steps
            // sum into accumulators of their own, so four products are independent of one another at any time
            uint32_t a[2][4], b[2][4];
            float s2[2][4];
            s2[0][0] = s2[0][1] = s2[0][2] = s2[0][3] = s2[1][0] = s2[1][1] = s2[1][2] = s2[1][3] = 0.f;
            ldmatrix_x4(smem_u32(qb), a[0][0], a[0][1], a[0][2], a[0][3]);
            ldmatrix_x4(smem_u32(kr), b[0][0], b[0][1], b[0][2], b[0][3]);
            int kk = 0;
            for (; kk + 1 < ksteps; kk += 2) {
                ldmatrix_x4(smem_u32(qb + (kk + 1) * 32), a[1][0], a[1][1], a[1][2], a[1][3]);
                ldmatrix_x4(smem_u32(kr + (kk + 1) * 32), b[1][0], b[1][1], b[1][2], b[1][3]);
                mma_bf16(s[0], a[0][0], a[0][1], a[0][2], a[0][3], b[0][0], b[0][1]);
                mma_bf16(s[1], a[0][0], a[0][1], a[0][2], a[0][3], b[0][2], b[0][3]);
                if (kk + 2 < ksteps) {
                    ldmatrix_x4(smem_u32(qb + (kk + 2) * 32), a[0][0], a[0][1], a[0][2], a[0][3]);
                    ldmatrix_x4(smem_u32(kr + (kk + 2) * 32), b[0][0], b[0][1], b[0][2], b[0][3]);
                }
                mma_bf16(s2[0], a[1][0], a[1][1], a[1][2], a[1][3], b[1][0], b[1][1]);
                mma_bf16(s2[1], a[1][0], a[1][1], a[1][2], a[1][3], b[1][2], b[1][3]);
            }
            if (kk < ksteps) {
                mma_bf16(s[0], a[0][0], a[0][1], a[0][2], a[0][3], b[0][0], b[0][1]);
                mma_bf16(s[1], a[0][0], a[0][1], a[0][2], a[0][3], b[0][2], b[0][3]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] += s2[j][e];
        }
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kpos = kb + wq * 16 + j * 8 + 2 * c + (e & 1);
                const int qpos = (e < 2) ? qpos_lo : qpos_hi;
                const bool seen = kpos < kend && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window);
                if (!seen) s[j][e] = -INFINITY;
            }
            mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        if (c == 0) {
            my_max[wq * 16 + r_lo] = mx_lo;
            my_max[wq * 16 + r_hi] = mx_hi;
        }
        __syncthreads();                                    // the four warps' row maxima of this tile are in
        float t_lo = fmaxf(fmaxf(my_max[r_lo], my_max[16 + r_lo]), fmaxf(my_max[32 + r_lo], my_max[48 + r_lo]));
        float t_hi = fmaxf(fmaxf(my_max[r_hi], my_max[16 + r_hi]), fmaxf(my_max[32 + r_hi], my_max[48 + r_hi]));
        // running maxima in scaled (log2) units: the scale is positive, so the order is the same
        const float mn_lo = fmaxf(m_lo, t_lo * sl2), mn_hi = fmaxf(m_hi, t_hi * sl2);
        const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float al_lo = exp2f(m_lo - base_lo), al_hi = exp2f(m_hi - base_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = exp2f(fmaf(s[j][0], sl2, -base_lo));
            s[j][1] = exp2f(fmaf(s[j][1], sl2, -base_lo));
            s[j][2] = exp2f(fmaf(s[j][2], sl2, -base_hi));
            s[j][3] = exp2f(fmaf(s[j][3], sl2, -base_hi));
            sum_lo += s[j][0] + s[j][1];
            sum_hi += s[j][2] + s[j][3];
            const int col = wq * 16 + j * 8 + 2 * c;
            *reinterpret_cast<uint32_t*>(pb + ((size_t)r_lo * PSTRIDE + col) * 2) = pack_bf16(s[j][0], s[j][1]);
            *reinterpret_cast<uint32_t*>(pb + ((size_t)r_hi * PSTRIDE + col) * 2) = pack_bf16(s[j][2], s[j][3]);
        }
        sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
        sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
        sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
        sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
        if (c == 0) {
            my_sum[wq * 16 + r_lo] = sum_lo;
            my_sum[wq * 16 + r_hi] = sum_hi;
        }
#pragma unroll
        for (int j = 0; j < VT; ++j) {
            o[j][0] *= al_lo;
            o[j][1] *= al_lo;
            o[j][2] *= al_hi;
            o[j][3] *= al_hi;
        }
        __syncthreads();                                    // the weights of all 64 keys and the row sums are in
        l_lo = l_lo * al_lo + ((my_sum[r_lo] + my_sum[16 + r_lo]) + (my_sum[32 + r_lo] + my_sum[48 + r_lo]));
        l_hi = l_hi * al_hi + ((my_sum[r_hi] + my_sum[16 + r_hi]) + (my_sum[32 + r_hi] + my_sum[48 + r_hi]));

        // ---- o += p . v over this warp's value columns
        const int vcol0 = wq * VT * 8;
#pragma unroll
        for (int k16 = 0; k16 < BN / 16; ++k16) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(smem_u32(pb + ((size_t)(lane & 15) * PSTRIDE + k16 * 16 + ((lane >> 4) << 3)) * 2), a0, a1, a2, a3);
            const unsigned char* vr = kt + (size_t)(k16 * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * rowb + (size_t)(vcol0 + ((lane >> 4) << 3)) * 2;
#pragma unroll
            for (int jp = 0; jp < VT / 2; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(smem_u32(vr + jp * 32), b0, b1, b2, b3);
                mma_bf16(o[2 * jp], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[2 * jp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    }

    // ---- results: each warp writes its value columns of its 16 rows
    const int vcol0 = wq * VT * 8;
    if (DECODE && a.splits > 1) {
        // m in natural-log units of the scaled score, as the combine kernel expects
        const float mo_lo = m_lo == -INFINITY ? -INFINITY : m_lo * 0.6931471805599453f;
        const float mo_hi = m_hi == -INFINITY ? -INFINITY : m_hi * 0.6931471805599453f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int gr = half ? gr_hi : gr_lo;
            if (gr >= nrows) continue;
            const size_t base = ((size_t)req * a.heads + gr) * a.splits + blockIdx.z;
#pragma unroll
            for (int j = 0; j < VT; ++j) {
                const int col = vcol0 + j * 8 + 2 * c;
                if (col < a.rank) a.part_o[base * a.rank + col] = o[j][half * 2];
                if (col + 1 < a.rank) a.part_o[base * a.rank + col + 1] = o[j][half * 2 + 1];
            }
            if (wq == 0 && c == 0) {
                a.part_ml[base * 2] = half ? mo_hi : mo_lo;
                a.part_ml[base * 2 + 1] = half ? l_hi : l_lo;
            }
        }
        return;
    }
    const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
    for (int j = 0; j < VT; ++j) {
        const int col = vcol0 + j * 8 + 2 * c;
        if (col >= a.rank) continue;                        // rank is even: a pair of columns is in or out together
        if (gr_lo < nrows)
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)tok0 * a.heads + gr_lo) * a.rank + col) = pack_bf16(o[j][0] * inv_lo, o[j][1] * inv_lo);
        if (gr_hi < nrows)
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)tok0 * a.heads + gr_hi) * a.rank + col) = pack_bf16(o[j][2] * inv_hi, o[j][3] * inv_hi);
    }
}

static int value_tiles(int rank) { return rank <= 128 ? 4 : (rank <= 256 ? 8 : (rank <= 384 ? 12 : 16)); }

static int row_stride(int row, int rank) {
    const int vt = value_tiles(rank);
    int cols = (row + 15) / 16 * 16;
    if (cols < 4 * vt * 8) cols = 4 * vt * 8;
    return cols + 8;                                        // an odd number of 16-byte pieces: ldmatrix without bank conflicts
}

static size_t smem_bytes(int rowp) {
    return (size_t)(ROWS + 2 * BN) * rowp * 2 + (size_t)2 * 16 * PSTRIDE * 2 + 2 * 2 * 4 * 16 * sizeof(float);
}

template <bool DECODE>
static int launch(const Args& a, dim3 grid, cudaStream_t stream) {
    const size_t smem = smem_bytes(a.rowp);
#define CASE(N)                                                                                                       \
    case N: {                                                                                                         \
        auto kern = latent_attention_kernel<N, DECODE>;                                                               \
        static size_t granted = 47 * 1024;      /* beside the kernel's static shared memory; set once per size */      \
        if (smem > granted) {                                                                                         \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
            if (e != cudaSuccess) { set_error("latent attention: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); return 2; } \
            granted = smem;                                                                                           \
        }                                                                                                             \
        kern<<<grid, THREADS, smem, stream>>>(a);                                                                     \
        break;                                                                                                        \
    }
    switch (value_tiles(a.rank)) {
        CASE(4) CASE(8) CASE(12) CASE(16)
        default: set_error("latent attention: rank %d", a.rank); return 1;
    }
#undef CASE
    return 0;
}

}  // namespace latent
}  // namespace lily

using namespace lily;
using namespace lily::latent;

// Whether the tensor-core kernel takes these sizes: rows of whole 16-byte pieces, an even rank of up to 512, tiles that
// fit the shared memory of a block.
LILY_API int lily_latent_attention_mma_takes(int row, int rank) {
    if (row <= 0 || rank <= 0 || rank > row || row % 8 != 0 || rank % 2 != 0 || rank > 512) return 0;
    return smem_bytes(row_stride(row, rank)) <= 220 * 1024 ? 1 : 0;
}

// New tokens a prefill tile holds for this many heads (the kernel's blocks take 32 of the tile's (token, head) rows each).
LILY_API int lily_latent_attention_mma_tile_tokens(int heads) { return heads >= ROWS ? 1 : ROWS / heads; }

LILY_API int lily_latent_attention_prefill_mma(const void* q, const void* cache, void* out, const int* block_table,
                                               int bt_stride, const int* cu_seqlens, const int* prefix_lens,
                                               const int* tile_req, const int* tile_start, int tiles, int tile_tokens,
                                               int heads, int row, int rank, int page_size, int window, float scale,
                                               cudaStream_t stream) {
    if (tiles == 0) return 0;
    LILY_REQUIRE(lily_latent_attention_mma_takes(row, rank), "latent attention: rows of %d with rank %d are not for this kernel", row, rank);
    LILY_REQUIRE(heads > 0 && tile_tokens > 0 && page_size > 0, "latent attention: heads=%d tile=%d page=%d", heads, tile_tokens, page_size);
    Args a{};
    a.q = (const __nv_bfloat16*)q; a.cache = (const __nv_bfloat16*)cache; a.out = (__nv_bfloat16*)out;
    a.block_table = block_table; a.bt_stride = bt_stride; a.cu_seqlens = cu_seqlens; a.prefix_lens = prefix_lens;
    a.tile_req = tile_req; a.tile_start = tile_start; a.splits = 1; a.heads = heads; a.row = row; a.rank = rank;
    a.page_size = page_size; a.window = window; a.tile_tokens = tile_tokens; a.rowp = row_stride(row, rank); a.scale = scale;
    dim3 grid(tiles, (tile_tokens * heads + ROWS - 1) / ROWS);
    LILY_REQUIRE(grid.y <= 65535, "latent attention: %d heads", heads);
    if (int rc = launch<false>(a, grid, stream)) return rc;
    LILY_CHECK_LAUNCH("latent_attention_prefill");
    return 0;
}

LILY_API int lily_latent_attention_decode_mma(const void* q, const void* cache, void* out, const int* block_table,
                                              int bt_stride, const int* seq_lens, float* scratch, int requests, int splits,
                                              int heads, int row, int rank, int page_size, int window, float scale,
                                              cudaStream_t stream) {
    if (requests == 0) return 0;
    LILY_REQUIRE(lily_latent_attention_mma_takes(row, rank), "latent attention: rows of %d with rank %d are not for this kernel", row, rank);
    LILY_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || scratch), "latent attention: %d key ranges need scratch", splits);
    Args a{};
    a.q = (const __nv_bfloat16*)q; a.cache = (const __nv_bfloat16*)cache; a.out = (__nv_bfloat16*)out;
    a.block_table = block_table; a.bt_stride = bt_stride; a.seq_lens = seq_lens; a.splits = splits; a.heads = heads;
    a.row = row; a.rank = rank; a.page_size = page_size; a.window = window; a.tile_tokens = 1;
    a.rowp = row_stride(row, rank); a.scale = scale;
    a.part_o = scratch;
    a.part_ml = scratch ? scratch + (size_t)requests * heads * splits * rank : nullptr;
    dim3 grid(requests, (heads + ROWS - 1) / ROWS, splits);
    if (int rc = launch<true>(a, grid, stream)) return rc;
    LILY_CHECK_LAUNCH("latent_attention_decode");
    return 0;
}

// 0, or 1 + the block of the first wait for a key tile that gave up (then cleared).  Synchronises the device.
LILY_API int lily_latent_attention_status() {
    int v = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, latent::g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(latent::g_status, &zero, sizeof(int));
    return v;
}
