// Risk scorer kernels (sm_100a).
//
// Replaces RiskScorer.score_prefill / score_with_attn (kvquant/scorer.py:385-416) and the
// mean-query attention of _expected_core_internals (kvquant/scorer.py:302-315).  Three streaming
// sweeps per (sample, KV head), each split over several CTAs:
//   1. K only:  logits of the G mean queries, |k|^2, per-split softmax statistics;
//   2. V:       p = mean_g softmax_g, |v|^2, partial sums of p v (for o) and of p;
//   3. V again: |v - o|^2 and the score; per-sample maximum for the sink slots.
// A quad of lanes owns one token (32 coordinates per lane, interleaved in 16-byte pieces so that a
// quad reads 64 contiguous bytes per instruction); each reduction takes two shuffles.  The next row
// of a lane is in flight while the current one is processed.
#include "common.cuh"

namespace odmkv {

constexpr int kScoreThreads = 256;
constexpr int kTokPerIter = kScoreThreads / 4;  // tokens per CTA iteration
constexpr int kMaxG = 16;

struct ScoreWs {
    float *logits;    // [BH, G, Tc]
    float *pbar;      // [BH, Tc]
    float *kn2;       // [BH, Tc]
    float *vn2;       // [BH, Tc]
    float *part_ml;   // [BH, nsplit, G, 2]
    float *part_o;    // [BH, nsplit, 128]
    float *part_ps;   // [BH, nsplit]
    unsigned *smax;   // [B]
    unsigned *status; // [1] set to 1 when a bounded wait of a sweep expired
};

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline int score_splits(int BH, int Tc) {
    int want = (6 * 148 + BH - 1) / BH;   // two waves of three CTAs per SM
    int by_len = (Tc + 511) / 512;
    int n = want < by_len ? want : by_len;
    if (n < 1) n = 1;
    if (n > 64) n = 64;
    return n;
}

inline size_t score_ws_layout(int B, int H, int G, int T, int n_sink, ScoreWs *ws, unsigned char *base) {
    const size_t BH = (size_t)B * H, Tc = (size_t)(T > n_sink ? T - n_sink : 0);
    const int ns = score_splits((int)BH, (int)Tc);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    size_t o_logits = take(BH * G * Tc * 4), o_pbar = take(BH * Tc * 4), o_kn2 = take(BH * Tc * 4), o_vn2 = take(BH * Tc * 4);
    size_t o_ml = take(BH * ns * G * 2 * 4), o_po = take(BH * ns * kD * 4), o_ps = take(BH * ns * 4), o_sm = take((size_t)B * 4 + 4);
    if (ws && base) {
        ws->logits = (float *)(base + o_logits); ws->pbar = (float *)(base + o_pbar); ws->kn2 = (float *)(base + o_kn2);
        ws->vn2 = (float *)(base + o_vn2); ws->part_ml = (float *)(base + o_ml); ws->part_o = (float *)(base + o_po);
        ws->part_ps = (float *)(base + o_ps); ws->smax = (unsigned *)(base + o_sm); ws->status = ws->smax + B;
    }
    return off;
}

// A quad of lanes owns one row.  Lane q of the quad holds the 16-byte pieces q, q + 4, q + 8, ... of
// the row, so the four lanes of a quad read 64 contiguous bytes with one instruction.  x[i] of lane q is
// coordinate coord_of<DT>(q, i).
template <int DT>
struct RawRow {
    static constexpr int kVec = (DT == kF32) ? 8 : 4;
    uint4 v[kVec];
};

template <int DT>
__device__ __forceinline__ int coord_of(int q, int i) {
    if constexpr (DT == kF32) return 16 * (i >> 2) + 4 * q + (i & 3);
    else return 32 * (i >> 3) + 8 * q + (i & 7);
}

template <int DT>
__device__ __forceinline__ void load_raw(const void *base, size_t row, int q, RawRow<DT> &r) {
    const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const unsigned char *>(base) +
                                                     row * kD * sizeof(typename Elem<DT>::T));
#pragma unroll
    for (int v = 0; v < RawRow<DT>::kVec; ++v) r.v[v] = __ldg(p + 4 * v + q);
}

template <int DT>
__device__ __forceinline__ void unpack_row(const RawRow<DT> &r, bool live, float (&x)[32]) {
    if (!live) {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = 0.f;
        return;
    }
#pragma unroll
    for (int v = 0; v < RawRow<DT>::kVec; ++v) {
        const uint32_t w[4] = {r.v[v].x, r.v[v].y, r.v[v].z, r.v[v].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if constexpr (DT == kF32) {
                x[4 * v + k] = __uint_as_float(w[k]);
            } else if constexpr (DT == kF16) {
                float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
                x[8 * v + 2 * k] = f.x; x[8 * v + 2 * k + 1] = f.y;
            } else {
                float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[k]));
                x[8 * v + 2 * k] = f.x; x[8 * v + 2 * k + 1] = f.y;
            }
        }
    }
}

// this lane's 32 entries of a 128-vector in shared memory, in the lane's coordinate order
template <int DT>
__device__ __forceinline__ void gather_lane_vec(const float *__restrict__ vec, int q, float (&o)[32]) {
    constexpr int kRun = (DT == kF32) ? 4 : 8;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        float4 f = *reinterpret_cast<const float4 *>(vec + coord_of<DT>(q, i));
        o[i] = f.x; o[i + 1] = f.y; o[i + 2] = f.z; o[i + 3] = f.w;
    }
    (void)kRun;
}

// ---- row stream: bulk asynchronous copies (TMA, one-dimensional) of 64-row tiles into a ring of shared-memory
// stages.  Thread 0 issues `cp.async.bulk` for a tile and arms the stage's mbarrier with the byte count; every
// thread waits on the barrier's phase before reading the stage.  A stage is refilled right after the CTA-wide
// barrier that ends its consumption, so kRingStages - 1 tiles (48 KB) are always in flight per CTA, independent
// of what the compiler does with the consuming code.  Waits are bounded: when one expires the CTA records it in
// the status word, waits (bounded again) for its outstanding copies and leaves.
constexpr int kRingStages = 4;    // K sweep: three CTAs per SM
constexpr int kRingStagesV = 6;   // V sweeps: two CTAs per SM, so more stages each keep the same bytes in flight
constexpr int kRingStageBytes = 16384;
constexpr unsigned kWaitPolls = 1u << 16;   // each poll blocks for up to the hardware's try_wait window

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity) {
    const uint32_t addr = smem_u32(bar);
    for (unsigned it = 0; it < kWaitPolls; ++it) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

template <int DT, int RING = kRingStages>
struct RowStream {
    static constexpr int kRowBytes = kD * (int)sizeof(typename Elem<DT>::T);
    static constexpr int kTileRows = kTokPerIter;                      // one row per quad and tile
    static constexpr int kTileBytes = kTileRows * kRowBytes;           // 16 KB (16-bit) or 32 KB (fp32)
    static constexpr int kStages = RING * kRingStageBytes / kTileBytes;
    unsigned char *ring;
    uint64_t *bars;
    const unsigned char *src;   // first row of this CTA
    int nrows, ntiles;

    __device__ void issue(int tile) {   // thread 0 only
        const int s = tile % kStages;
        const int rows = min(kTileRows, nrows - tile * kTileRows);
        const uint32_t bytes = (uint32_t)rows * kRowBytes;
        const uint32_t bar = smem_u32(bars + s), dst = smem_u32(ring + (size_t)s * kTileBytes);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                     ::"r"(dst), "l"(src + (size_t)tile * kTileBytes), "r"(bytes), "r"(bar) : "memory");
    }
    __device__ void start(unsigned char *ring_, uint64_t *bars_, const void *base, size_t first_row, int nrows_) {
        ring = ring_; bars = bars_; nrows = nrows_;
        src = reinterpret_cast<const unsigned char *>(base) + first_row * kRowBytes;
        ntiles = (nrows + kTileRows - 1) / kTileRows;
        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s)
                asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(bars + s)) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int t = 0; t < kStages && t < ntiles; ++t) issue(t);
    }
    // all threads; false when the wait expired (uniform over the CTA)
    __device__ bool acquire(int tile, unsigned *status) {
        const bool ok = mbar_wait(bars + tile % kStages, (unsigned)(tile / kStages) & 1u);
        if (__syncthreads_or(!ok)) {
            if (threadIdx.x == 0) {
                atomicExch(status, 1u);
                // outstanding copies target this CTA's shared memory: give them a bounded chance to land
                for (int t = tile; t < ntiles && t < tile + kStages; ++t) mbar_wait(bars + t % kStages, (unsigned)(t / kStages) & 1u);
            }
            __syncthreads();
            return false;
        }
        return true;
    }
    __device__ const unsigned char *row_ptr(int tile, int row_in_tile) const {
        return ring + (size_t)(tile % kStages) * kTileBytes + (size_t)row_in_tile * kRowBytes;
    }
    // after the consumers are done with `tile` (call from all threads)
    __device__ void release(int tile) {
        __syncthreads();
        if (threadIdx.x == 0 && tile + kStages < ntiles) issue(tile + kStages);
    }
};

// load this lane's pieces of a row that sits in shared memory
template <int DT>
__device__ __forceinline__ void load_raw_smem(const unsigned char *row, int q, RawRow<DT> &r) {
    const uint4 *p = reinterpret_cast<const uint4 *>(row);
#pragma unroll
    for (int v = 0; v < RawRow<DT>::kVec; ++v) r.v[v] = p[4 * v + q];
}

__device__ inline float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

// ---- sweep 1 ---------------------------------------------------------------------------------
// GM: compile-time bound on the group size (4, 8 or 16).  Lane q of a quad keeps the running softmax
// statistics of the query heads g with g % 4 == q.
template <int DT, int GM>
__global__ void __launch_bounds__(kScoreThreads, 3) score_logits_kernel(const void *__restrict__ K, const float *__restrict__ mu,
                                                                         int H, int G, int T, int n_sink, int nsplit, ScoreWs ws) {
    extern __shared__ __align__(128) unsigned char score_ring[];
    __shared__ __align__(8) uint64_t bars[kRingStages];
    __shared__ __align__(16) float mus[GM * kD];
    __shared__ float red_m[GM][kTokPerIter], red_l[GM][kTokPerIter];
    const int bh = blockIdx.y, split = blockIdx.x, b = bh / H;
    const int Tc = T - n_sink;
    const int tid = threadIdx.x, q = tid & 3, quad = tid >> 2, warp = tid >> 5, lane = tid & 31;
    const float inv_sqrt_d = 1.0f / sqrtf((float)kD);
    for (int i = tid; i < GM * kD; i += kScoreThreads)
        mus[i] = i < G * kD ? mu[((size_t)b * H * G + (size_t)(bh % H) * G) * kD + i] : 0.f;
    __syncthreads();
    const int per = (Tc + nsplit - 1) / nsplit;
    const int j0 = split * per, j1 = min(Tc, j0 + per);
    float m_run[GM / 4], l_run[GM / 4];
#pragma unroll
    for (int k = 0; k < GM / 4; ++k) { m_run[k] = -INFINITY; l_run[k] = 0.f; }
    const size_t row_base = (size_t)bh * T + n_sink;
    RowStream<DT> rs;
    rs.start(score_ring, bars, K, row_base + j0, max(j1 - j0, 0));
    // every lane of a warp runs the same number of iterations: the quad reductions below are
    // full-warp shuffles and must not be reached by a partial warp
    for (int tile = 0; tile < rs.ntiles; ++tile) {
        if (!rs.acquire(tile, ws.status)) return;
        const int j = j0 + tile * kTokPerIter + quad;
        const bool live = j < j1;
        float x[32];
        {
            RawRow<DT> raw;
            if (live) load_raw_smem<DT>(rs.row_ptr(tile, quad), q, raw);
            unpack_row<DT>(raw, live, x);
        }
        rs.release(tile);
        float kk = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) kk = fmaf(x[i], x[i], kk);
        kk = quad_sum(kk);
        if (q == 0 && live) ws.kn2[(size_t)bh * Tc + j] = kk;
#pragma unroll
        for (int g = 0; g < GM; ++g) {
            if (g < G) {
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 m4 = *reinterpret_cast<const float4 *>(mus + g * kD + coord_of<DT>(q, i));
                    acc = fmaf(x[i], m4.x, acc);
                    acc = fmaf(x[i + 1], m4.y, acc);
                    acc = fmaf(x[i + 2], m4.z, acc);
                    acc = fmaf(x[i + 3], m4.w, acc);
                }
                acc = quad_sum(acc) * inv_sqrt_d;
                if ((g & 3) == q && live) {
                    ws.logits[((size_t)bh * G + g) * Tc + j] = acc;
                    const float mo = m_run[g >> 2];
                    const float mn = fmaxf(mo, acc);
                    const float e = expf(fminf(mo, acc) - mn);
                    l_run[g >> 2] = acc > mo ? fmaf(l_run[g >> 2], e, 1.0f) : l_run[g >> 2] + e;
                    m_run[g >> 2] = mn;
                }
            }
        }
    }
    // block merge of the per-quad (m, l) pairs: warp w reduces the heads w, w + 8
#pragma unroll
    for (int k = 0; k < GM / 4; ++k) {
        red_m[4 * k + q][quad] = m_run[k];
        red_l[4 * k + q][quad] = l_run[k];
    }
    __syncthreads();
    for (int g = warp; g < G; g += kScoreThreads / 32) {
        const float ma = red_m[g][lane], mb = red_m[g][lane + 32];
        const float mm = warp_max(fmaxf(ma, mb));
        float l = 0.f;
        if (mm > -INFINITY) {
            if (red_l[g][lane] > 0.f) l += red_l[g][lane] * expf(ma - mm);
            if (red_l[g][lane + 32] > 0.f) l += red_l[g][lane + 32] * expf(mb - mm);
        }
        l = warp_sum(l);
        if (lane == 0) {
            float *dst = ws.part_ml + (((size_t)bh * nsplit + split) * G + g) * 2;
            dst[0] = mm; dst[1] = l;
        }
    }
}

// ---- sweep 1 on the tensor cores (16-bit caches, G <= 8) ----------------------------------------
// logits^T = mu . K^T as m16n8k16 products: the sixteen A rows are the fp16 (bf16) high limbs of the G mean
// queries (rows 0..7) and their low limbs (rows 8..15), so the product carries about 22 (16) bits of mu; the
// eight B columns are the eight rows a warp holds, one per quad.  Contraction index p of k-block kb stands for
// coordinate 8 (4 (kb / 2) + t) + 4 (kb % 2) + {0, 1 | 2, 3} of lane t's pieces, which makes the B registers
// the lane's raw 32-bit words, unconverted.  |k|^2 stays an fp32 FMA sum.
template <int DT>
__device__ __forceinline__ void mma_16816_f32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (DT == kF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int DT>
__device__ __forceinline__ void split_pair(float v0, float v1, uint32_t &hi, uint32_t &lo) {
    if constexpr (DT == kF16) {
        const __half h0 = __float2half_rn(v0), h1 = __float2half_rn(v1);
        const __half l0 = __float2half_rn(v0 - __half2float(h0)), l1 = __float2half_rn(v1 - __half2float(h1));
        hi = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
        lo = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
    } else {
        const __nv_bfloat16 h0 = __float2bfloat16_rn(v0), h1 = __float2bfloat16_rn(v1);
        const __nv_bfloat16 l0 = __float2bfloat16_rn(v0 - __bfloat162float(h0)), l1 = __float2bfloat16_rn(v1 - __bfloat162float(h1));
        hi = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
        lo = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
    }
}

template <int DT>
__global__ void __launch_bounds__(kScoreThreads, 3) score_logits_mma_kernel(const void *__restrict__ K, const float *__restrict__ mu,
                                                                             int H, int G, int T, int n_sink, int nsplit, ScoreWs ws) {
    static_assert(DT != kF32, "16-bit caches only");
    extern __shared__ __align__(128) unsigned char score_ring[];
    __shared__ __align__(8) uint64_t bars[kRingStages];
    __shared__ float red_m[8][kScoreThreads / 32], red_l[8][kScoreThreads / 32];
    const int bh = blockIdx.y, split = blockIdx.x, b = bh / H;
    const int Tc = T - n_sink;
    const int tid = threadIdx.x, q = tid & 3, quad = tid >> 2, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2;
    const float inv_sqrt_d = 1.0f / sqrtf((float)kD);
    // A fragments of this lane: head g8, high limbs in a0 / a2, low limbs in a1 / a3
    uint32_t afr[8][4];
    {
        const float *mrow = mu + ((size_t)b * H * G + (size_t)(bh % H) * G + (g8 < G ? g8 : 0)) * kD;
#pragma unroll
        for (int kb = 0; kb < 8; ++kb) {
            const int d0 = 8 * (4 * (kb >> 1) + q) + 4 * (kb & 1);
            float4 m4 = *reinterpret_cast<const float4 *>(mrow + d0);
            if (g8 >= G) m4 = make_float4(0.f, 0.f, 0.f, 0.f);
            split_pair<DT>(m4.x, m4.y, afr[kb][0], afr[kb][1]);
            split_pair<DT>(m4.z, m4.w, afr[kb][2], afr[kb][3]);
        }
    }
    const int per = (Tc + nsplit - 1) / nsplit;
    const int j0 = split * per, j1 = min(Tc, j0 + per);
    float m_run = -INFINITY, l_run = 0.f;   // head g8, rows 2q and 2q + 1 of every group of eight
    const size_t row_base = (size_t)bh * T + n_sink;
    RowStream<DT> rs;
    rs.start(score_ring, bars, K, row_base + j0, max(j1 - j0, 0));
    for (int tile = 0; tile < rs.ntiles; ++tile) {
        if (!rs.acquire(tile, ws.status)) return;
        const int j = j0 + tile * kTokPerIter + quad;
        const bool live = j < j1;
        RawRow<DT> raw;
        if (live) load_raw_smem<DT>(rs.row_ptr(tile, quad), q, raw);
        else {
#pragma unroll
            for (int v = 0; v < 4; ++v) raw.v[v] = make_uint4(0u, 0u, 0u, 0u);
        }
        rs.release(tile);
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        float kk = 0.f;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint32_t w[4] = {raw.v[v].x, raw.v[v].y, raw.v[v].z, raw.v[v].w};
            mma_16816_f32<DT>(d, afr[2 * v], w[0], w[1]);
            mma_16816_f32<DT>(d, afr[2 * v + 1], w[2], w[3]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 f;
                if constexpr (DT == kF16) f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
                else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[k]));
                kk = fmaf(f.x, f.x, kk);
                kk = fmaf(f.y, f.y, kk);
            }
        }
        kk = quad_sum(kk);
        if (q == 0 && live) ws.kn2[(size_t)bh * Tc + j] = kk;
        // this lane's two logits: head g8, rows 2q and 2q + 1 of the warp's eight rows
        const int jr = j0 + tile * kTokPerIter + warp * 8 + 2 * q;
        if (g8 < G) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (jr + e < j1) {
                    const float acc = (d[e] + d[2 + e]) * inv_sqrt_d;
                    ws.logits[((size_t)bh * G + g8) * Tc + jr + e] = acc;
                    const float mn = fmaxf(m_run, acc);
                    const float ex = expf(fminf(m_run, acc) - mn);
                    l_run = acc > m_run ? fmaf(l_run, ex, 1.0f) : l_run + ex;
                    m_run = mn;
                }
            }
        }
    }
    // merge over the four lanes of a head, then over the warps
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m_run, o), lo = __shfl_xor_sync(0xffffffffu, l_run, o);
        const float mn = fmaxf(m_run, mo);
        float l = 0.f;
        if (l_run > 0.f) l += l_run * expf(m_run - mn);
        if (lo > 0.f) l += lo * expf(mo - mn);
        m_run = mn; l_run = l;
    }
    if (q == 0) { red_m[g8][warp] = m_run; red_l[g8][warp] = l_run; }
    __syncthreads();
    if (tid < G) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kScoreThreads / 32; ++w) mm = fmaxf(mm, red_m[tid][w]);
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < kScoreThreads / 32; ++w)
            if (red_l[tid][w] > 0.f) l += red_l[tid][w] * expf(red_m[tid][w] - mm);
        float *dst = ws.part_ml + (((size_t)bh * nsplit + split) * G + tid) * 2;
        dst[0] = mm; dst[1] = l;
    }
}

// merge the split statistics of one (b, h): final max and denominator per query head
__device__ inline void merge_ml(const float *__restrict__ part_ml, int bh, int nsplit, int G, float *M, float *L) {
    // called by threads g < G
    const int g = threadIdx.x;
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(((size_t)bh * nsplit + s) * G + g) * 2]);
    float l = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float *p = part_ml + (((size_t)bh * nsplit + s) * G + g) * 2;
        if (p[1] > 0.f) l += p[1] * expf(p[0] - m);
    }
    M[g] = m; L[g] = l;
}

// ---- sweep 2 ---------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kScoreThreads, 2) score_pv_kernel(const void *__restrict__ V, int H, int G, int T, int n_sink,
                                                                     int nsplit, ScoreWs ws) {
    extern __shared__ __align__(128) unsigned char score_ring[];
    __shared__ __align__(8) uint64_t bars[kRingStagesV];
    __shared__ float M[kMaxG], L[kMaxG];
    __shared__ float osum[kTokPerIter / 8][kD];  // one row per warp
    __shared__ float psum[kTokPerIter / 8];
    const int bh = blockIdx.y, split = blockIdx.x;
    const int Tc = T - n_sink;
    const int tid = threadIdx.x, q = tid & 3, quad = tid >> 2, warp = tid >> 5, lane = tid & 31;
    if (tid < G) merge_ml(ws.part_ml, bh, nsplit, G, M, L);
    __syncthreads();
    const int per = (Tc + nsplit - 1) / nsplit;
    const int j0 = split * per, j1 = min(Tc, j0 + per);
    float o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = 0.f;
    float ps = 0.f;
    const float inv_g = 1.0f / (float)G;
    const size_t row_base = (size_t)bh * T + n_sink;
    RowStream<DT, kRingStagesV> rs;
    rs.start(score_ring, bars, V, row_base + j0, max(j1 - j0, 0));
    // lane q adds the softmax terms of the heads g = q, q + 4, ...; their logits are fetched one tile ahead
    float lg_n[kMaxG / 4];
    auto fetch_logits = [&](int j) {
#pragma unroll
        for (int k = 0; k < kMaxG / 4; ++k) {
            const int g = q + 4 * k;
            lg_n[k] = (j < j1 && g < G) ? __ldg(ws.logits + ((size_t)bh * G + g) * Tc + j) : 0.f;
        }
    };
    fetch_logits(j0 + quad);
    for (int tile = 0; tile < rs.ntiles; ++tile) {
        if (!rs.acquire(tile, ws.status)) return;
        const int j = j0 + tile * kTokPerIter + quad;
        const bool live = j < j1;
        float x[32];
        {
            RawRow<DT> raw;
            if (live) load_raw_smem<DT>(rs.row_ptr(tile, quad), q, raw);
            unpack_row<DT>(raw, live, x);
        }
        rs.release(tile);
        float lg[kMaxG / 4];
#pragma unroll
        for (int k = 0; k < kMaxG / 4; ++k) lg[k] = lg_n[k];
        fetch_logits(j + kTokPerIter);
        float p = 0.f;
        if (live) {
#pragma unroll
            for (int k = 0; k < kMaxG / 4; ++k) {
                const int g = q + 4 * k;
                if (g < G) p += expf(lg[k] - M[g]) / L[g];
            }
        }
        p = quad_sum(p) * inv_g;
        float vv = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) { vv = fmaf(x[i], x[i], vv); o[i] = fmaf(p, x[i], o[i]); }
        vv = quad_sum(vv);
        if (q == 0 && live) {
            ws.pbar[(size_t)bh * Tc + j] = p;
            ws.vn2[(size_t)bh * Tc + j] = vv;
            ps += p;
        }
    }
    // reduce over the 8 quads of a warp (lanes with equal q), then over warps through shared memory
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float v = o[i];
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        o[i] = v;
    }
    ps += __shfl_xor_sync(0xffffffffu, ps, 4);
    ps += __shfl_xor_sync(0xffffffffu, ps, 8);
    ps += __shfl_xor_sync(0xffffffffu, ps, 16);
    if (lane < 4) {
#pragma unroll
        for (int i = 0; i < 32; ++i) osum[warp][coord_of<DT>(lane, i)] = o[i];
        if (lane == 0) psum[warp] = ps;
    }
    __syncthreads();
    if (tid < kD) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kTokPerIter / 8; ++w) v += osum[w][tid];
        ws.part_o[((size_t)bh * nsplit + split) * kD + tid] = v;
    }
    if (tid == 0) {
        float v = 0.f;
        for (int w = 0; w < kTokPerIter / 8; ++w) v += psum[w];
        ws.part_ps[(size_t)bh * nsplit + split] = v;
    }
}

// ---- sweep 3 ---------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kScoreThreads, 2) score_final_kernel(const void *__restrict__ V, int H, int T, int n_sink,
                                                                        int nsplit, float eps, ScoreWs ws, float *__restrict__ scores) {
    extern __shared__ __align__(128) unsigned char score_ring[];
    __shared__ __align__(8) uint64_t bars[kRingStagesV];
    __shared__ __align__(16) float ob[kD];
    __shared__ float wmax[kScoreThreads / 32];
    const int bh = blockIdx.y, split = blockIdx.x, b = bh / H;
    const int Tc = T - n_sink;
    const int tid = threadIdx.x, q = tid & 3, quad = tid >> 2, warp = tid >> 5, lane = tid & 31;
    if (tid < kD) {
        float v = 0.f, ps = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            v += ws.part_o[((size_t)bh * nsplit + s) * kD + tid];
            ps += ws.part_ps[(size_t)bh * nsplit + s];
        }
        ob[tid] = v / fmaxf(ps, 1e-8f);
    }
    __syncthreads();
    float oq[32];
    gather_lane_vec<DT>(ob, q, oq);
    const int per = (Tc + nsplit - 1) / nsplit;
    const int j0 = split * per, j1 = min(Tc, j0 + per);
    float best = 0.f;
    const size_t row_base = (size_t)bh * T + n_sink;
    RowStream<DT, kRingStagesV> rs;
    rs.start(score_ring, bars, V, row_base + j0, max(j1 - j0, 0));
    // the three per-row scalars of the next tile are fetched one tile ahead by the lane that uses them
    float pb_n = 0.f, vn_n = 0.f, kn_n = 0.f;
    auto fetch_scalars = [&](int j) {
        if (q == 0 && j < j1) {
            const size_t e = (size_t)bh * Tc + j;
            pb_n = __ldg(ws.pbar + e); vn_n = __ldg(ws.vn2 + e); kn_n = __ldg(ws.kn2 + e);
        }
    };
    fetch_scalars(j0 + quad);
    for (int tile = 0; tile < rs.ntiles; ++tile) {
        if (!rs.acquire(tile, ws.status)) return;
        const int j = j0 + tile * kTokPerIter + quad;
        const bool live = j < j1;
        float x[32];
        {
            RawRow<DT> raw;
            if (live) load_raw_smem<DT>(rs.row_ptr(tile, quad), q, raw);
            unpack_row<DT>(raw, live, x);
        }
        rs.release(tile);
        const float pb = pb_n, vn = vn_n, kn = kn_n;
        fetch_scalars(j + kTokPerIter);
        float ir = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) { float dlt = x[i] - oq[i]; ir = fmaf(dlt, dlt, ir); }
        ir = quad_sum(ir);
        if (q == 0 && live) {
            float p = pb + eps;
            float s = p * p * (vn + (kn / (float)kD) * ir);
            scores[(size_t)bh * T + n_sink + j] = s;
            best = fmaxf(best, s);  // NaN-free inputs assumed; scores are non-negative
        }
    }
    best = warp_max(best);
    if (lane == 0) wmax[warp] = best;
    __syncthreads();
    if (tid == 0) {
        float v = wmax[0];
        for (int w = 1; w < kScoreThreads / 32; ++w) v = fmaxf(v, wmax[w]);
        atomicMax(ws.smax + b, __float_as_uint(v));  // order-preserving for non-negative floats
    }
}

__global__ void score_sinks_kernel(float *__restrict__ scores, const unsigned *__restrict__ smax, int H, int T, int n_sink) {
    const int bh = blockIdx.x;
    if ((int)threadIdx.x < n_sink) scores[(size_t)bh * T + threadIdx.x] = __uint_as_float(smax[bh / H]);
}

__global__ void fill_ones_kernel(float *__restrict__ p, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = 1.0f;
}

// ---- score_with_attn: one CTA per row of T <= 1024 tokens ---------------------------------------
template <int DT>
__global__ void __launch_bounds__(kScoreThreads) score_with_attn_kernel(const void *__restrict__ K, const void *__restrict__ V,
                                                                         const float *__restrict__ p, int T, float eps,
                                                                         float *__restrict__ scores) {
    __shared__ float osum[kScoreThreads / 32][kD];
    __shared__ float psum[kScoreThreads / 32];
    __shared__ __align__(16) float ob[kD];
    const int row = blockIdx.x;
    const int tid = threadIdx.x, q = tid & 3, quad = tid >> 2, warp = tid >> 5, lane = tid & 31;
    float o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = 0.f;
    float ps = 0.f;
    for (int j = quad; j < T; j += kTokPerIter) {
        float x[32];
        RawRow<DT> rv;
        load_raw<DT>(V, (size_t)row * T + j, q, rv);
        unpack_row<DT>(rv, true, x);
        float pj = p[(size_t)row * T + j];
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = fmaf(pj, x[i], o[i]);
        if (q == 0) ps += pj;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float v = o[i];
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        o[i] = v;
    }
    ps += __shfl_xor_sync(0xffffffffu, ps, 4);
    ps += __shfl_xor_sync(0xffffffffu, ps, 8);
    ps += __shfl_xor_sync(0xffffffffu, ps, 16);
    if (lane < 4) {
#pragma unroll
        for (int i = 0; i < 32; ++i) osum[warp][coord_of<DT>(lane, i)] = o[i];
        if (lane == 0) psum[warp] = ps;
    }
    __syncthreads();
    if (tid < kD) {
        float v = 0.f, s = 0.f;
        for (int w = 0; w < kScoreThreads / 32; ++w) { v += osum[w][tid]; s += psum[w]; }
        ob[tid] = v / fmaxf(s, 1e-8f);
    }
    __syncthreads();
    float oq[32];
    gather_lane_vec<DT>(ob, q, oq);
    for (int jb = 0; jb < T; jb += kTokPerIter) {
        const int j = jb + quad;
        const bool live = j < T;
        float x[32], y[32];
        RawRow<DT> rv, rk;
        if (live) {
            load_raw<DT>(V, (size_t)row * T + j, q, rv);
            load_raw<DT>(K, (size_t)row * T + j, q, rk);
        }
        unpack_row<DT>(rv, live, x);
        unpack_row<DT>(rk, live, y);
        float ir = 0.f, vv = 0.f, kk = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float dlt = x[i] - oq[i];
            ir = fmaf(dlt, dlt, ir);
            vv = fmaf(x[i], x[i], vv);
            kk = fmaf(y[i], y[i], kk);
        }
        ir = quad_sum(ir); vv = quad_sum(vv); kk = quad_sum(kk);
        if (q == 0 && live) {
            float pe = p[(size_t)row * T + j] + eps;
            scores[(size_t)row * T + j] = pe * pe * (vv + (kk / (float)kD) * ir);
        }
    }
}

}  // namespace odmkv

using namespace odmkv;

extern "C" {

size_t odmkv_score_workspace_bytes(int B, int H, int G, int T) {
    if (B <= 0 || H <= 0 || G <= 0 || T <= 0) return 0;
    return score_ws_layout(B, H, G, T, 0, nullptr, nullptr) + 256;
}

// byte offset, inside a score workspace, of the 32-bit word that a sweep sets to 1 when one of its bounded waits
// on a bulk copy expired (the scores of that call are then invalid); 0 after a clean call
size_t odmkv_score_status_offset(int B, int H, int G, int T, int n_sink) {
    if (B <= 0 || H <= 0 || G <= 0 || T <= n_sink) return 0;
    ScoreWs ws;
    unsigned char *base = reinterpret_cast<unsigned char *>(256);   // any non-null base: only differences are used
    score_ws_layout(B, H, G, T, n_sink, &ws, base);
    return (size_t)(reinterpret_cast<unsigned char *>(ws.status) - base);
}

int odmkv_score_prefill(const void *K, const void *V, int dtype, const float *mu, int B, int H, int G, int T,
                        int n_sink, float eps, float *scores, void *workspace, size_t workspace_bytes,
                        void *stream) {
    if (!K || !V || !mu || !scores) return ODMKV_ERR_ARG;
    if (B <= 0 || H <= 0 || G <= 0 || G > kMaxG || T <= 0 || n_sink < 0 || n_sink > 32 || (long long)B * H > 65535) return ODMKV_ERR_SHAPE;
    if (dtype < 0 || dtype > 2) return ODMKV_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (T <= n_sink) {
        size_t n = (size_t)B * H * T;
        fill_ones_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(scores, n);
        return launch_status();
    }
    if (!workspace) return ODMKV_ERR_ARG;
    if (((uintptr_t)workspace & 255) != 0) return ODMKV_ERR_WORKSPACE;
    if ((((uintptr_t)K | (uintptr_t)V) & 15) != 0) return ODMKV_ERR_ARG;   // rows are sources of 16-byte aligned bulk copies
    ScoreWs ws;
    size_t need = score_ws_layout(B, H, G, T, n_sink, &ws, (unsigned char *)workspace);
    if (workspace_bytes < need) return ODMKV_ERR_WORKSPACE;
    const int BH = B * H, Tc = T - n_sink, ns = score_splits(BH, Tc);
    cudaMemsetAsync(ws.smax, 0, (size_t)B * 4 + 4, st);   // per-sample maxima and the status word
    dim3 grid(ns, BH);
    constexpr int kRing = kRingStages * kRingStageBytes, kRingV = kRingStagesV * kRingStageBytes;
    timing_begin("score", st);
#define ODMKV_SCORE_L(DT, GM)                                                                                         \
    {                                                                                                                 \
        cudaError_t e = cudaFuncSetAttribute(score_logits_kernel<DT, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing); \
        if (e != cudaSuccess) return (int)e;                                                                          \
        score_logits_kernel<DT, GM><<<grid, kScoreThreads, kRing, st>>>(K, mu, H, G, T, n_sink, ns, ws);              \
    }
#define ODMKV_SCORE_M(DT)                                                                                             \
    {                                                                                                                 \
        cudaError_t e = cudaFuncSetAttribute(score_logits_mma_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing); \
        if (e != cudaSuccess) return (int)e;                                                                          \
        score_logits_mma_kernel<DT><<<grid, kScoreThreads, kRing, st>>>(K, mu, H, G, T, n_sink, ns, ws);              \
    }
#define ODMKV_SCORE(DT)                                                                                               \
    if (G <= 4) ODMKV_SCORE_L(DT, 4) else if (G <= 8) ODMKV_SCORE_L(DT, 8) else ODMKV_SCORE_L(DT, 16)                 \
    ODMKV_SCORE_REST(DT)
#define ODMKV_SCORE16(DT)                                                                                             \
    if (G <= 8) ODMKV_SCORE_M(DT) else ODMKV_SCORE_L(DT, 16)                                                          \
    ODMKV_SCORE_REST(DT)
#define ODMKV_SCORE_REST(DT)                                                                                          \
    {                                                                                                                 \
        cudaError_t e = cudaFuncSetAttribute(score_pv_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingV); \
        if (e != cudaSuccess) return (int)e;                                                                          \
        e = cudaFuncSetAttribute(score_final_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingV);        \
        if (e != cudaSuccess) return (int)e;                                                                          \
        score_pv_kernel<DT><<<grid, kScoreThreads, kRingV, st>>>(V, H, G, T, n_sink, ns, ws);                         \
        score_final_kernel<DT><<<grid, kScoreThreads, kRingV, st>>>(V, H, T, n_sink, ns, eps, ws, scores);            \
    }
    if (dtype == kF16) { ODMKV_SCORE16(kF16) } else if (dtype == kBF16) { ODMKV_SCORE16(kBF16) } else { ODMKV_SCORE(kF32) }
#undef ODMKV_SCORE
#undef ODMKV_SCORE16
#undef ODMKV_SCORE_REST
#undef ODMKV_SCORE_M
#undef ODMKV_SCORE_L
    timing_end(st);
    if (n_sink > 0) score_sinks_kernel<<<BH, 32, 0, st>>>(scores, ws.smax, H, T, n_sink);
    return launch_status();
}

int odmkv_score_with_attn(const void *K, const void *V, int dtype, const float *p, int R, int T, float eps,
                          float *scores, void *stream) {
    if (!K || !V || !p || !scores) return ODMKV_ERR_ARG;
    if (R <= 0 || T <= 0 || T > 1024) return ODMKV_ERR_SHAPE;
    if (dtype < 0 || dtype > 2) return ODMKV_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == kF16) score_with_attn_kernel<kF16><<<R, kScoreThreads, 0, st>>>(K, V, p, T, eps, scores);
    else if (dtype == kBF16) score_with_attn_kernel<kBF16><<<R, kScoreThreads, 0, st>>>(K, V, p, T, eps, scores);
    else score_with_attn_kernel<kF32><<<R, kScoreThreads, 0, st>>>(K, V, p, T, eps, scores);
    return launch_status();
}

}  // extern "C"
