// Column statistics of causal softmax attention on the fifth-generation tensor cores (sm_100a: tcgen05.mma with
// both operands in shared memory and the accumulator in tensor memory).
//
// Replaces _chunked_attention_qk (kvquant/attention_utils.py:160-211): for queries r = 0..Tq-1 of every query head and
// keys j = 0..Tkv-1 of its KV head, logits q_r.k_j / scale with keys j > r + q_offset masked out (the reference masks
// q_pos < k_pos, i.e. q_offset = 0), softmax over the keys per query, mean over the G query heads of a KV head, and
// per key the sum, the maximum and the sum of squares of that mean over all queries.  The sum divided by the number of
// queries that see a key is the attention weight RiskScorer.score_with_attn expects (kvquant/scorer.py:406-416).
//
// Two passes, both plain TN products of 128-row tiles with K = 128 (the head dimension):
//   pass 1 (rows = queries): S = Q K^T per (query head, 128 queries) over the visible key tiles; the thread that owns
//          a query row reads it from tensor memory and keeps the running maximum and sum: log2-sum-exp per query;
//   pass 2 (rows = keys):    S^T = K Q^T per (KV head, 128 keys) over blocks of RB queries x G heads as the N
//          dimension; the thread that owns a key reads its row, turns it into probabilities with the stored
//          log-sum-exps, averages the G heads of each query in registers and accumulates the three statistics --
//          no exchange between threads, no atomics: a CTA owns its keys.
// Operand tiles are copied by the threads (cp.async, 16 bytes each) into the canonical K-major layout without
// swizzle: 8-row x 16-byte core matrices, 128 bytes between K-neighbours, 2048 bytes between row groups.
// The exponentials bound both passes (one per logit and pass on the special-function unit), not the products.
// Every wait on an mbarrier is bounded; an expired wait sets the status word and the CTA runs out without waiting
// again, releasing its tensor memory.
#include "common.cuh"

namespace odmkv {

namespace {

constexpr int kWThreads = 128;
constexpr int kWRows = 128;                       // rows of the A tile = tensor-memory lanes
constexpr uint32_t kLbo = 128, kSbo = 2048;       // bytes between K-adjacent core matrices / between 8-row groups
constexpr int kTileBytes = kWRows * kD * 2;       // 32 KiB per 128 rows
constexpr unsigned kPolls = 1u << 12;
constexpr unsigned kSuspendNs = 1000000u;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMasked = -1.0e30f;

struct WinArgs {
    const void *Q, *K;
    float *lse2;            // [B * Hq, Tq] log2-sum-exp of the scaled logits
    float *sum_attn, *max_attn, *sum_sq;   // [B * H, Tkv]
    unsigned *status;
    int B, H, G, Tq, Tkv, q_offset, RB;
    float c;                // log2(e) / scale
    int bf16;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ float ex2f(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x)); return y; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;    // zero-fill when the row does not exist
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((kLbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((kSbo >> 4) & 0x3FFF) << 32) |
           (1ull << 46);
}
// instruction descriptor: fp32 accumulator, A and B fp16 or bf16, both K-major, M = 128
__device__ __forceinline__ uint32_t idesc_f16(int N, int bf16) {
    return (1u << 4) | ((uint32_t)bf16 << 7) | ((uint32_t)bf16 << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred P1;\nelect.sync _|P1, 0xffffffff;\nselp.u32 %0, 1, 0, P1;\n}\n" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ bool mbar_poll(uint32_t bar, unsigned parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(kSuspendNs) : "memory");
    return ok != 0;
}
// bounded wait: false when it expired (the caller stops issuing work and reports through the status word)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, unsigned parity) {
    for (unsigned it = 0; it < kPolls; ++it)
        if (mbar_poll(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Copy `groups` groups of eight rows into the canonical layout at `tile`: piece (row 8 gi + tid % 8, 16-byte chunk
// c) lands at gi * 2048 + c * 128 + (tid % 8) * 16, so the 32 stores of a warp fill 512 consecutive bytes.
// row_ptr(row) returns the row's address in global memory, or nullptr for a row that does not exist: such a row is
// zero-filled (a copy of zero source bytes, which still names a valid global address, `any_row`).
template <class RowPtr>
__device__ __forceinline__ void stage_rows(unsigned char *tile, int groups, int tid, const unsigned char *any_row, RowPtr row_ptr) {
    const int r8 = tid & 7, c0 = tid >> 3;       // 16 chunk columns: every thread takes chunk c0 of one row per group
    for (int gi = 0; gi < groups; ++gi) {
        const unsigned char *src = reinterpret_cast<const unsigned char *>(row_ptr(gi * 8 + r8));
        const uint32_t dst = smem_u32(tile) + gi * kSbo + c0 * kLbo + r8 * 16;
        cp_async16(dst, src ? src + c0 * 16 : any_row, src != nullptr);
    }
}

// one 128 x N x 128 product into tensor memory: eight K = 16 steps, 256 bytes apart in both tiles
__device__ __forceinline__ void issue_product(uint32_t tmem, const unsigned char *a_tile, const unsigned char *b_tile, int N, int bf16,
                                              uint32_t bar) {
    const uint32_t idesc = idesc_f16(N, bf16);
    const uint32_t a0 = smem_u32(a_tile), b0 = smem_u32(b_tile);
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) umma_f16(tmem, smem_desc(a0 + ks * 256), smem_desc(b0 + ks * 256), idesc, ks ? 1u : 0u);
    umma_commit(bar);
}

__device__ __forceinline__ uint32_t tmem_alloc(uint32_t *slot, int cols, int warp) {
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"((uint32_t)cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    return *slot;
}
__device__ __forceinline__ void tmem_free(uint32_t base, int cols, int warp) {
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"((uint32_t)cols) : "memory");
}

// ---- pass 1: log2-sum-exp per (query head, query) -----------------------------------------------------------------
// grid: (ceil(Tq / 128), B * Hq); shared memory: Q tile + two K tiles
__global__ void __launch_bounds__(kWThreads) win_lse_kernel(const WinArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
    unsigned char *q_tile = smem, *k_tiles = smem + kTileBytes;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int Hq = a.H * a.G;
    const int bq = blockIdx.y, b = bq / Hq, hq = bq % Hq, h = hq / a.G;
    const int r0 = blockIdx.x * kWRows;
    const size_t esz = 2;
    const unsigned char *Qb = reinterpret_cast<const unsigned char *>(a.Q) + ((size_t)bq * a.Tq) * kD * esz;
    const unsigned char *Kb = reinterpret_cast<const unsigned char *>(a.K) + ((size_t)(b * a.H + h) * a.Tkv) * kD * esz;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_s = 0;
    }
    const uint32_t tmem = tmem_alloc(&tmem_slot, 128, warp);
    const uint32_t tmem_lane = tmem + ((uint32_t)(warp * 32) << 16);

    // keys this query tile can see: j <= r + q_offset for its last row
    const int r_last = min(r0 + kWRows, a.Tq) - 1;
    const int n_keys = max(0, min(a.Tkv, r_last + a.q_offset + 1));
    const int n_kt = (n_keys + kWRows - 1) / kWRows;
    stage_rows(q_tile, 16, tid, Qb, [&](int row) { return r0 + row < a.Tq ? Qb + (size_t)(r0 + row) * kD * esz : nullptr; });
    auto stage_k = [&](int kt) {
        stage_rows(k_tiles + (kt & 1) * kTileBytes, 16, tid, Kb,
                   [&](int row) { return kt * kWRows + row < a.Tkv ? Kb + (size_t)(kt * kWRows + row) * kD * esz : nullptr; });
    };
    if (n_kt > 0) stage_k(0);
    cp_async_commit();

    const int r = r0 + tid;
    const int vis = r + a.q_offset;          // last visible key of this row
    float m = kMasked, l = 0.f;
    bool dead = false;
    for (int kt = 0; kt < n_kt; ++kt) {
        if (kt + 1 < n_kt) stage_k(kt + 1);
        cp_async_commit();
        cp_async_wait<1>();
        proxy_fence();
        __syncthreads();
        dead = dead || abort_s != 0;
        if (warp == 0 && !dead) {
            tc_fence_after();
            if (elect_one()) issue_product(tmem, q_tile, k_tiles + (kt & 1) * kTileBytes, 128, a.bf16, smem_u32(&bar));
            __syncwarp();
        }
        if (!dead && !mbar_wait(smem_u32(&bar), (unsigned)(kt & 1))) {
            dead = true;
            abort_s = 1;
            atomicExch(a.status, 1u);
        }
        dead = __any_sync(0xffffffffu, dead);   // the tensor-memory loads below are warp-wide instructions
        tc_fence_after();
        if (!dead) {
            const int j0 = kt * kWRows;
            // two sweeps over the row: maximum first, then one exponential per visible logit
            float tile_max = kMasked;
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t v[32];
                tmem_ld32(tmem_lane + cb * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int j = j0 + cb * 32 + i;
                    if (j <= vis && j < a.Tkv) tile_max = fmaxf(tile_max, __uint_as_float(v[i]) * a.c);
                }
            }
            // (every thread of a warp takes both sweeps: the tensor-memory loads are warp-wide; a row that sees no key
            //  of this tile adds nothing and keeps its maximum)
            const float m_new = fmaxf(m, tile_max);
            float acc = 0.f;
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t v[32];
                tmem_ld32(tmem_lane + cb * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int j = j0 + cb * 32 + i;
                    if (j <= vis && j < a.Tkv) acc += ex2f(fmaf(__uint_as_float(v[i]), a.c, -m_new));
                }
            }
            l = l * ex2f(m - m_new) + acc;
            m = m_new;
        }
        tc_fence_before();
        __syncthreads();   // the accumulator and this K buffer are free again
    }
    cp_async_wait<0>();
    if (r < a.Tq) a.lse2[(size_t)bq * a.Tq + r] = l > 0.f ? m + log2f(l) : -kMasked;   // no visible key: every probability 0
    tmem_free(tmem, 128, warp);
}

// ---- pass 2: sum / max / sum of squares per key of the head-averaged probabilities -------------------------------
// grid: (ceil(Tkv / 128), B * H); shared memory: K tile + two query blocks of RB * G rows + their log-sum-exps
template <int RB>
__global__ void __launch_bounds__(kWThreads) win_cols_kernel(const WinArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
    const int G = a.G, N = RB * G;
    const int blk_bytes = N * kD * 2;
    unsigned char *k_tile = smem, *q_blks = smem + kTileBytes;
    float *lse_s = reinterpret_cast<float *>(smem + kTileBytes + 2 * blk_bytes);   // [2][N]
    const int tid = threadIdx.x, warp = tid >> 5;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int Hq = a.H * G;
    const int j0 = blockIdx.x * kWRows;
    const size_t esz = 2;
    const unsigned char *Kb = reinterpret_cast<const unsigned char *>(a.K) + ((size_t)bh * a.Tkv) * kD * esz;
    const unsigned char *Qb = reinterpret_cast<const unsigned char *>(a.Q) + ((size_t)(b * Hq + h * G) * a.Tq) * kD * esz;
    const float *lse_b = a.lse2 + (size_t)(b * Hq + h * G) * a.Tq;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_s = 0;
    }
    const uint32_t tmem = tmem_alloc(&tmem_slot, 256, warp);
    const uint32_t tmem_lane = tmem + ((uint32_t)(warp * 32) << 16);

    stage_rows(k_tile, 16, tid, Kb, [&](int row) { return j0 + row < a.Tkv ? Kb + (size_t)(j0 + row) * kD * esz : nullptr; });
    // query blocks that can see a key of this tile: r + q_offset >= j0
    const int n_rb = (a.Tq + RB - 1) / RB;
    const int rb_first = max(0, j0 - a.q_offset) / RB;
    auto stage_q = [&](int rb) {
        const int buf = (rb - rb_first) & 1;
        // row n = g * RB + rr of the block is query rb * RB + rr of head g
        stage_rows(q_blks + buf * blk_bytes, N / 8, tid, Qb, [&](int row) {
            const int g = row / RB, rr = rb * RB + row % RB;
            return rr < a.Tq ? Qb + ((size_t)g * a.Tq + rr) * kD * esz : nullptr;
        });
        for (int n = tid; n < N; n += kWThreads) {
            const int g = n / RB, rr = rb * RB + n % RB;
            lse_s[buf * N + n] = rr < a.Tq ? lse_b[(size_t)g * a.Tq + rr] : -kMasked;
        }
    };
    if (rb_first < n_rb) stage_q(rb_first);
    cp_async_commit();

    const int j = j0 + tid;
    const float inv_g = 1.0f / (float)G;
    float s_sum = 0.f, s_max = 0.f, s_sq = 0.f;
    bool dead = false;
    for (int rb = rb_first; rb < n_rb; ++rb) {
        const int it = rb - rb_first, buf = it & 1;
        if (rb + 1 < n_rb) stage_q(rb + 1);
        cp_async_commit();
        cp_async_wait<1>();
        proxy_fence();
        __syncthreads();
        dead = dead || abort_s != 0;
        if (warp == 0 && !dead) {
            tc_fence_after();
            if (elect_one()) issue_product(tmem, k_tile, q_blks + buf * blk_bytes, N, a.bf16, smem_u32(&bar));
            __syncwarp();
        }
        if (!dead && !mbar_wait(smem_u32(&bar), (unsigned)(it & 1))) {
            dead = true;
            abort_s = 1;
            atomicExch(a.status, 1u);
        }
        dead = __any_sync(0xffffffffu, dead);   // the tensor-memory loads below are warp-wide instructions
        tc_fence_after();
        if (!dead) {
            float mean[RB];
#pragma unroll
            for (int i = 0; i < RB; ++i) mean[i] = 0.f;
            const float *ls = lse_s + buf * N;
            const int r_base = rb * RB;
            for (int g = 0; g < G; ++g) {
                uint32_t v[RB];
                if constexpr (RB == 32) tmem_ld32(tmem_lane + g * RB, reinterpret_cast<uint32_t(&)[32]>(v));
                else tmem_ld16(tmem_lane + g * RB, reinterpret_cast<uint32_t(&)[16]>(v));
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < RB; ++i) {
                    // key j is visible to query r when j <= r + q_offset; queries past Tq carry a huge log-sum-exp
                    const float p = (j <= r_base + i + a.q_offset) ? ex2f(fmaf(__uint_as_float(v[i]), a.c, -ls[g * RB + i])) : 0.f;
                    mean[i] += p;
                }
            }
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                const float mg = mean[i] * inv_g;
                s_sum += mg;
                s_max = fmaxf(s_max, mg);
                s_sq = fmaf(mg, mg, s_sq);
            }
        }
        tc_fence_before();
        __syncthreads();
    }
    cp_async_wait<0>();
    if (j < a.Tkv) {
        const size_t o = (size_t)bh * a.Tkv + j;
        a.sum_attn[o] = s_sum;
        a.max_attn[o] = s_max;
        a.sum_sq[o] = s_sq;
    }
    tmem_free(tmem, 256, warp);
}

int pick_rb(int G) { return 32 * G <= 256 ? 32 : 16; }

size_t lse_bytes(int B, int H, int G, int Tq) { return (((size_t)B * H * G * Tq * sizeof(float)) + 255) & ~(size_t)255; }

}  // namespace

}  // namespace odmkv

using namespace odmkv;

extern "C" {

size_t odmkv_window_stats_workspace_bytes(int B, int H, int G, int Tq) {
    if (B <= 0 || H <= 0 || G <= 0 || Tq <= 0) return 0;
    return lse_bytes(B, H, G, Tq) + 256;
}

size_t odmkv_window_stats_status_offset(int B, int H, int G, int Tq) { return lse_bytes(B, H, G, Tq); }

int odmkv_window_attn_stats(const void *Q, const void *K, int dtype, int B, int H, int G, int Tq, int Tkv, int q_offset, float scale,
                            float *sum_attn, float *max_attn, float *sum_sq_attn, void *workspace, size_t workspace_bytes,
                            void *stream) {
    if (!Q || !K || !sum_attn || !max_attn || !sum_sq_attn || !workspace) return ODMKV_ERR_ARG;
    if (B <= 0 || H <= 0 || G <= 0 || Tq <= 0 || Tkv <= 0 || q_offset < 0 || !(scale > 0.f)) return ODMKV_ERR_SHAPE;
    if (dtype != kF16 && dtype != kBF16) return ODMKV_ERR_UNSUPPORTED;
    if (G > 16) return ODMKV_ERR_UNSUPPORTED;                       // N = 16 G columns must fit one product (256)
    if ((((uintptr_t)Q | (uintptr_t)K) & 15) != 0) return ODMKV_ERR_ARG;   // rows are copied 16 bytes at a time
    if (workspace_bytes < odmkv_window_stats_workspace_bytes(B, H, G, Tq)) return ODMKV_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    WinArgs a;
    a.Q = Q; a.K = K;
    a.lse2 = reinterpret_cast<float *>(workspace);
    a.status = reinterpret_cast<unsigned *>(reinterpret_cast<unsigned char *>(workspace) + lse_bytes(B, H, G, Tq));
    a.sum_attn = sum_attn; a.max_attn = max_attn; a.sum_sq = sum_sq_attn;
    a.B = B; a.H = H; a.G = G; a.Tq = Tq; a.Tkv = Tkv; a.q_offset = q_offset; a.RB = pick_rb(G);
    a.c = kLog2e / scale; a.bf16 = dtype == kBF16 ? 1 : 0;
    cudaError_t e = cudaMemsetAsync(a.status, 0, 256, st);
    if (e != cudaSuccess) return (int)e;
    const int smem1 = 3 * kTileBytes;
    const int N = a.RB * G;
    const int smem2 = kTileBytes + 2 * N * kD * 2 + 2 * N * (int)sizeof(float);
    e = cudaFuncSetAttribute(win_lse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
    if (e != cudaSuccess) return (int)e;
    timing_begin("window_lse", st);
    win_lse_kernel<<<dim3((Tq + kWRows - 1) / kWRows, B * H * G), kWThreads, smem1, st>>>(a);
    timing_end(st);
    timing_begin("window_cols", st);
    if (a.RB == 32) {
        e = cudaFuncSetAttribute(win_cols_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
        if (e != cudaSuccess) return (int)e;
        win_cols_kernel<32><<<dim3((Tkv + kWRows - 1) / kWRows, B * H), kWThreads, smem2, st>>>(a);
    } else {
        e = cudaFuncSetAttribute(win_cols_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
        if (e != cudaSuccess) return (int)e;
        win_cols_kernel<16><<<dim3((Tkv + kWRows - 1) / kWRows, B * H), kWThreads, smem2, st>>>(a);
    }
    timing_end(st);
    return launch_status();
}

}  // extern "C"
