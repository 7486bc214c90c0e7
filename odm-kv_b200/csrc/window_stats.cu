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
// Operand tiles sit in shared memory in the K-major layout with the 128-byte swizzle: a tile of R rows is two blocks
// of R x 128 bytes (coordinates 0-63 and 64-127), row r of a block at r * 128, its 16-byte chunk c at position
// c ^ (r % 8).  A tile arrives as two tensor copies (TMA, cp.async.bulk.tensor, boxes of 64 coordinates x R rows --
// for pass 2 x G heads -- of the row-major global tensor; rows past the end read as zeros); a first version with the
// unswizzled layout needed 16-byte rows in its boxes and spent 2 300 clocks per tile in the copy engine.  Without the
// driver's tensor-map encoder the threads copy 16-byte pieces themselves (cp.async) into the same layout.
// The exponentials bound both passes (one per logit and pass on the special-function unit), not the products.
// Every wait on an mbarrier is bounded; an expired wait sets the status word and the CTA runs out without waiting
// again, releasing its tensor memory.
#include "common.cuh"

#include <cuda.h>
#include <cstring>

namespace odmkv {

namespace {

constexpr int kWThreads = 256;                    // two threads per tensor-memory lane: each takes half of the columns
constexpr int kWRows = 128;                       // rows of the A tile = tensor-memory lanes
constexpr uint32_t kSbo = 1024;                   // bytes between 8-row groups of a swizzled block (8 rows x 128 bytes)
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

struct WinMaps {
    CUtensorMap q_tile;     // box: 128 rows of one query head (pass 1)
    CUtensorMap q_blk;      // box: RB rows of each of the G heads of a KV head (pass 2)
    CUtensorMap k_tile;     // box: 128 rows of one KV head
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

// shared-memory matrix descriptor, K-major, 128-byte swizzle: start address, (unused) leading offset, 1024 bytes
// between 8-row groups, descriptor version 1, layout type 2
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)((kSbo >> 4) & 0x3FFF) << 32) | (1ull << 46) |
           (2ull << 61);
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, unsigned parity, const volatile int *abort_flag = nullptr) {
    for (unsigned it = 0; it < kPolls; ++it) {
        if (mbar_poll(bar, parity)) return true;
        if (abort_flag && *abort_flag) return false;
    }
    return false;
}
// one tensor copy of a box into shared memory, completion counted in bytes on an mbarrier
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int row, int head, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(row), "r"(head), "r"(bar) : "memory");
}
// both 64-coordinate blocks of a tile of `rows` rows (x = 0 and 64: 128-byte steps, as the copy engine requires)
__device__ __forceinline__ void tma_load_tile(unsigned char *tile, int rows, const CUtensorMap *map, int row, int head, uint32_t bar) {
    tma_load_3d(smem_u32(tile), map, 0, row, head, bar);
    tma_load_3d(smem_u32(tile) + rows * 128, map, 64, row, head, bar);
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
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

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}

// Thread copies of `groups` groups of eight rows into the swizzled layout of a tile of 8 * groups rows: the piece
// (row r, 16-byte chunk c) lands in block c / 8 at r * 128 + ((c % 8) ^ (r % 8)) * 16.  Two neighbouring lanes take
// the two halves of one 32-byte sector of a row, a warp eight rows x four chunks; warps 0-3 / 4-7 alternate groups.
// row_ptr(row) returns the row's address in global memory, or nullptr for a row that does not exist: such a row is
// zero-filled (a copy of zero source bytes, which still names a valid global address, `any_row`).
template <class RowPtr>
__device__ __forceinline__ void stage_rows(unsigned char *tile, int groups, int tid, const unsigned char *any_row, RowPtr row_ptr) {
    const int lane = tid & 31, warp = tid >> 5;
    const int r8 = (lane >> 1) & 7, c0 = (warp & 3) * 4 + (lane >> 4) * 2 + (lane & 1);
    const uint32_t blk = (uint32_t)(c0 >> 3) * (uint32_t)groups * 1024u + (uint32_t)(((c0 & 7) ^ r8) * 16);
    for (int gi = warp >> 2; gi < groups; gi += kWThreads / 128) {
        const unsigned char *src = reinterpret_cast<const unsigned char *>(row_ptr(gi * 8 + r8));
        const uint32_t dst = smem_u32(tile) + blk + (gi * 8 + r8) * 128;
        cp_async16(dst, src ? src + c0 * 16 : any_row, src != nullptr);
    }
}

// one 128 x N x 128 product into tensor memory: eight K = 16 steps, 32 bytes apart inside a 64-coordinate block
// (the swizzle is applied to the address bits by the hardware), the second block after the first
__device__ __forceinline__ void issue_product(uint32_t tmem, const unsigned char *a_tile, const unsigned char *b_tile, int N, int bf16,
                                              uint32_t bar) {
    const uint32_t idesc = idesc_f16(N, bf16);
    const uint32_t a0 = smem_u32(a_tile), b0 = smem_u32(b_tile);
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
        const uint32_t ao = (ks >> 2) * (kWRows * 128) + (ks & 3) * 32, bo = (ks >> 2) * (N * 128) + (ks & 3) * 32;
        umma_f16(tmem, smem_desc(a0 + ao), smem_desc(b0 + bo), idesc, ks ? 1u : 0u);
    }
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

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

constexpr int kWorkWarps = kWThreads / 32;           // warps that turn accumulators into statistics
constexpr int kTmaThreads = kWThreads + 32;          // plus one warp that drives the copies and the products

// ---- pass 1: log2-sum-exp per (query head, query) -----------------------------------------------------------------
// grid: (ceil(Tq / 128), B * Hq); shared memory: Q tile + two K tiles; tensor memory: two 128-column accumulators.
// Eight working warps: warp w reads tensor-memory lanes 32 (w % 4) .. +31 (a row each), warps 0-3 the first 64
// columns of a tile and warps 4-7 the last 64; the two partial (maximum, sum) pairs of a row meet once, at the end.
// With tensor copies (TMA = true) a ninth warp drives everything else: one of its lanes issues the copies two tiles
// ahead and the products one tile ahead, and the working warps only wait for "product kt done" and report
// "accumulator free" through mbarriers -- no block-wide barrier in the loop.  With thread copies (TMA = false) the
// eight warps copy, meet at one block-wide barrier per tile, and warp 0 issues the products.
template <bool TMA>
__global__ void __launch_bounds__(TMA ? kTmaThreads : kWThreads, 2) win_lse_kernel(const WinArgs a, const __grid_constant__ WinMaps maps) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t mma_bar[2];    // product kt arrives on mma_bar[kt & 1]
    __shared__ __align__(8) uint64_t full_bar[2];   // tensor copies: bytes of K tile kt land on full_bar[kt & 1]
    __shared__ __align__(8) uint64_t free_bar[2];   // the working warps are done with accumulator kt & 1
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
    __shared__ float2 part_s[kWRows];
    unsigned char *q_tile = smem, *k_tiles = smem + kTileBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, half = (warp >> 2) & 1;
    const int Hq = a.H * a.G;
    const int bq = blockIdx.y, b = bq / Hq, hq = bq % Hq, h = hq / a.G;
    const int r0 = blockIdx.x * kWRows;
    const size_t esz = 2;
    const unsigned char *Qb = reinterpret_cast<const unsigned char *>(a.Q) + ((size_t)bq * a.Tq) * kD * esz;
    const unsigned char *Kb = reinterpret_cast<const unsigned char *>(a.K) + ((size_t)(b * a.H + h) * a.Tkv) * kD * esz;
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&mma_bar[i], 1);
            mbar_init(&full_bar[i], 1);
            mbar_init(&free_bar[i], kWorkWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_s = 0;
    }
    const uint32_t tmem = tmem_alloc(&tmem_slot, 256, warp);
    const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + half * 64;

    // keys this query tile can see: j <= r + q_offset for its last row
    const int r_last = min(r0 + kWRows, a.Tq) - 1;
    const int n_keys = max(0, min(a.Tkv, r_last + a.q_offset + 1));
    const int n_kt = (n_keys + kWRows - 1) / kWRows;
    const int row = (warp & 3) * 32 + lane;
    const int r = r0 + row;
    const int vis = r + a.q_offset;          // last visible key of this row
    float m = kMasked, l = 0.f;

    // one accumulator -> running (maximum, sum) of this thread's half row
    auto epilogue = [&](int kt) {
        const int j0 = kt * kWRows + half * 64;
        const uint32_t acc_addr = tmem_lane + (kt & 1) * 128;
        // a tile every row of this CTA sees completely needs no mask (all but the last tiles of a row block)
        const bool open = kt * kWRows + kWRows - 1 <= r0 + a.q_offset && (kt + 1) * kWRows <= a.Tkv;
#pragma unroll 1
        for (int cb = 0; cb < 2; ++cb) {
            uint32_t v[32];
            tmem_ld32(acc_addr + cb * 32, v);
            tmem_ld_wait();
            float cmax = kMasked;
            if (open) {
#pragma unroll
                for (int i = 0; i < 32; ++i) cmax = fmaxf(cmax, __uint_as_float(v[i]));
                cmax *= a.c;
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int j = j0 + cb * 32 + i;
                    if (j <= vis && j < a.Tkv) cmax = fmaxf(cmax, __uint_as_float(v[i]) * a.c);
                }
            }
            const float m_new = fmaxf(m, cmax);
            float acc0 = 0.f, acc1 = 0.f;
            if (open) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    acc0 += ex2f(fmaf(__uint_as_float(v[i]), a.c, -m_new));
                    acc1 += ex2f(fmaf(__uint_as_float(v[i + 1]), a.c, -m_new));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int j = j0 + cb * 32 + i;
                    if (j <= vis && j < a.Tkv) acc0 += ex2f(fmaf(__uint_as_float(v[i]), a.c, -m_new));
                }
            }
            l = l * ex2f(m - m_new) + (acc0 + acc1);     // both at the masked value: factor 1, nothing added
            m = m_new;
        }
    };

    if constexpr (TMA) {
        if (warp == kWorkWarps) {
            if (lane == 0) {
                bool ok = true;
                auto load_k = [&](int kt) {
                    const uint32_t fb = smem_u32(&full_bar[kt & 1]);
                    mbar_expect_tx(fb, kt == 0 ? 2 * kTileBytes : kTileBytes);
                    if (kt == 0) tma_load_tile(q_tile, kWRows, &maps.q_tile, r0, bq, fb);
                    tma_load_tile(k_tiles + (kt & 1) * kTileBytes, kWRows, &maps.k_tile, kt * kWRows, b * a.H + h, fb);
                };
                if (n_kt > 0) load_k(0);
                if (n_kt > 1) load_k(1);
                for (int kt = 0; kt < n_kt && ok; ++kt) {
                    const int bsel = kt & 1;
                    const unsigned use = (unsigned)(kt >> 1);
                    if (kt >= 2) ok = mbar_wait(smem_u32(&free_bar[bsel]), (use - 1) & 1, &abort_s);      // epilogue kt - 2 done
                    if (ok) ok = mbar_wait(smem_u32(&full_bar[bsel]), use & 1, &abort_s);                 // K tile kt landed
                    if (!ok) break;
                    tc_fence_after();
                    issue_product(tmem + bsel * 128, q_tile, k_tiles + bsel * kTileBytes, 128, a.bf16, smem_u32(&mma_bar[bsel]));
                    if (kt + 2 < n_kt) {                                                                  // refill this K buffer
                        ok = mbar_wait(smem_u32(&mma_bar[bsel]), use & 1, &abort_s);
                        if (ok) load_k(kt + 2);
                    }
                }
                if (!ok) {
                    abort_s = 1;
                    atomicExch(a.status, 1u);
                }
            }
            __syncwarp();
        } else {
            for (int kt = 0; kt < n_kt; ++kt) {
                bool ok = mbar_wait(smem_u32(&mma_bar[kt & 1]), (unsigned)((kt >> 1) & 1), &abort_s);
                ok = __all_sync(0xffffffffu, ok);    // the tensor-memory loads are warp-wide instructions
                if (!ok) {
                    abort_s = 1;
                    atomicExch(a.status, 1u);
                    break;
                }
                tc_fence_after();
                epilogue(kt);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&free_bar[kt & 1]));
            }
        }
    } else {
        stage_rows(q_tile, 16, tid, Qb, [&](int row_) { return r0 + row_ < a.Tq ? Qb + (size_t)(r0 + row_) * kD * esz : nullptr; });
        auto stage_k = [&](int kt) {
            if (kt < n_kt)
                stage_rows(k_tiles + (kt & 1) * kTileBytes, 16, tid, Kb,
                           [&](int row_) { return kt * kWRows + row_ < a.Tkv ? Kb + (size_t)(kt * kWRows + row_) * kD * esz : nullptr; });
            cp_async_commit();
        };
        auto issue = [&](int kt) {   // warp 0, converged
            tc_fence_after();
            if (elect_one()) issue_product(tmem + (kt & 1) * 128, q_tile, k_tiles + (kt & 1) * kTileBytes, 128, a.bf16, smem_u32(&mma_bar[kt & 1]));
            __syncwarp();
        };
        stage_k(0);
        stage_k(1);
        cp_async_wait<1>();
        proxy_fence();
        __syncthreads();
        if (warp == 0 && n_kt > 0) issue(0);
        bool dead = false;
        for (int kt = 0; kt < n_kt; ++kt) {
            // Two products stay in flight: tile kt + 1 is issued before tile kt is awaited.  Its accumulator was read
            // during the previous iteration, hence the barrier first; every thread has waited for its own pieces of
            // K tile kt + 1.
            cp_async_wait<0>();
            proxy_fence();
            tc_fence_before();
            __syncthreads();
            dead = dead || abort_s != 0;
            if (warp == 0 && !dead && kt + 1 < n_kt) issue(kt + 1);
            if (!dead && !mbar_wait(smem_u32(&mma_bar[kt & 1]), (unsigned)((kt >> 1) & 1), &abort_s)) {
                dead = true;
                abort_s = 1;
                atomicExch(a.status, 1u);
            }
            stage_k(kt + 2);                        // product kt is complete: its K buffer takes tile kt + 2
            dead = __any_sync(0xffffffffu, dead);   // the tensor-memory loads below are warp-wide instructions
            tc_fence_after();
            if (!dead) epilogue(kt);
        }
        cp_async_wait<0>();
    }
    if (warp < kWorkWarps && half == 1) part_s[row] = make_float2(m, l);
    __syncthreads();
    if (warp < kWorkWarps && half == 0 && r < a.Tq) {
        const float2 o = part_s[row];
        const float mm = fmaxf(m, o.x);
        const float ll = l * ex2f(m - mm) + o.y * ex2f(o.x - mm);
        a.lse2[(size_t)bq * a.Tq + r] = ll > 0.f ? mm + log2f(ll) : -kMasked;   // no visible key: every probability 0
    }
    tmem_free(tmem, 256, warp);
}

// ---- pass 2: sum / max / sum of squares per key of the head-averaged probabilities -------------------------------
// grid: (ceil(Tkv / 128), B * H); shared memory: K tile + two query blocks of RB * G rows (+ four rows of their
// log-sum-exps for the thread-copy form); tensor memory: two accumulators of N = RB * G columns.  Working warps 0-3
// take the first RB / 2 queries of a block, warps 4-7 the others (every head of them); the two partial statistics of
// a key meet once, at the end.  Same two forms as pass 1, over query blocks.
template <int RB, bool TMA>
__global__ void __launch_bounds__(TMA ? kTmaThreads : kWThreads, 2) win_cols_kernel(const WinArgs a, const __grid_constant__ WinMaps maps) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t mma_bar[2];    // product `it` arrives on mma_bar[it & 1]
    __shared__ __align__(8) uint64_t full_bar[2];   // tensor copies: bytes of query block `it` land on full_bar[it & 1]
    __shared__ __align__(8) uint64_t free_bar[2];   // the working warps are done with accumulator it & 1
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
    __shared__ float part_s[3][kWRows];
    __shared__ __align__(16) float lse_w[TMA ? kWorkWarps : 1][2][128];   // tensor-copy form: per working warp, two blocks
    constexpr int HB = RB / 2;
    const int G = a.G, N = RB * G;
    const int blk_bytes = N * kD * 2;
    const int acc_stride = N <= 128 ? 128 : 256, tmem_cols = 2 * acc_stride;
    unsigned char *k_tile = smem, *q_blks = smem + kTileBytes;
    float *lse_s = reinterpret_cast<float *>(smem + kTileBytes + 2 * blk_bytes);   // [4][N], thread-copy form only
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, half = (warp >> 2) & 1;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int Hq = a.H * G;
    const int j0 = blockIdx.x * kWRows;
    const size_t esz = 2;
    const unsigned char *Kb = reinterpret_cast<const unsigned char *>(a.K) + ((size_t)bh * a.Tkv) * kD * esz;
    const unsigned char *Qb = reinterpret_cast<const unsigned char *>(a.Q) + ((size_t)(b * Hq + h * G) * a.Tq) * kD * esz;
    const float *lse_b = a.lse2 + (size_t)(b * Hq + h * G) * a.Tq;
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&mma_bar[i], 1);
            mbar_init(&full_bar[i], 1);
            mbar_init(&free_bar[i], kWorkWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_s = 0;
    }
    const uint32_t tmem = tmem_alloc(&tmem_slot, tmem_cols, warp);
    const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + half * HB;

    // query blocks that can see a key of this tile: r + q_offset >= j0
    const int n_rb = (a.Tq + RB - 1) / RB;
    const int rb_first = max(0, j0 - a.q_offset) / RB;
    const int n_it = max(0, n_rb - rb_first);
    const int row = (warp & 3) * 32 + lane;
    const int j = j0 + row;
    const float inv_g = 1.0f / (float)G;
    float s_sum = 0.f, s_max = 0.f, s_sq = 0.f;

    // one accumulator -> the three statistics of this thread's key over its half of the block's queries;
    // ls(g): log-sum-exps of head g for those queries (shared memory, or global memory for a whole block)
    auto epilogue = [&](int it, auto ls_of) {
        const int rb = rb_first + it;
        float mean[HB];
#pragma unroll
        for (int i = 0; i < HB; ++i) mean[i] = 0.f;
        const uint32_t acc_addr = tmem_lane + (it & 1) * acc_stride;
        const int r_base = rb * RB + half * HB;
        // a block whose first query already sees the last key of this tile needs no mask
        const bool open = j0 + kWRows - 1 <= rb * RB + a.q_offset;
        for (int g = 0; g < G; ++g) {
            uint32_t v[HB];
            if constexpr (HB == 16) tmem_ld16(acc_addr + g * RB, reinterpret_cast<uint32_t(&)[16]>(v));
            else tmem_ld8(acc_addr + g * RB, reinterpret_cast<uint32_t(&)[8]>(v));
            float lg[HB];
            ls_of(g, r_base, lg);
            tmem_ld_wait();
            if (open) {
#pragma unroll
                for (int i = 0; i < HB; ++i) mean[i] += ex2f(fmaf(__uint_as_float(v[i]), a.c, -lg[i]));
            } else {
#pragma unroll
                for (int i = 0; i < HB; ++i)   // key j is visible to query r when j <= r + q_offset
                    if (j <= r_base + i + a.q_offset) mean[i] += ex2f(fmaf(__uint_as_float(v[i]), a.c, -lg[i]));
            }
        }
#pragma unroll
        for (int i = 0; i < HB; ++i) {
            const float mg = mean[i] * inv_g;
            s_sum += mg;
            s_max = fmaxf(s_max, mg);
            s_sq = fmaf(mg, mg, s_sq);
        }
    };

    if constexpr (TMA) {
        if (warp == kWorkWarps) {
            if (lane == 0) {
                bool ok = true;
                auto load_q = [&](int it) {   // two copies: RB rows of each of the G heads (the first barrier also counts the K tile)
                    const uint32_t fb = smem_u32(&full_bar[it & 1]);
                    mbar_expect_tx(fb, (uint32_t)blk_bytes + (it == 0 ? (uint32_t)kTileBytes : 0u));
                    if (it == 0) tma_load_tile(k_tile, kWRows, &maps.k_tile, j0, bh, fb);
                    tma_load_tile(q_blks + (it & 1) * blk_bytes, N, &maps.q_blk, (rb_first + it) * RB, b * Hq + h * G, fb);
                };
                if (n_it > 0) load_q(0);
                if (n_it > 1) load_q(1);
                for (int it = 0; it < n_it && ok; ++it) {
                    const int bsel = it & 1;
                    const unsigned use = (unsigned)(it >> 1);
                    if (it >= 2) ok = mbar_wait(smem_u32(&free_bar[bsel]), (use - 1) & 1, &abort_s);
                    if (ok) ok = mbar_wait(smem_u32(&full_bar[bsel]), use & 1, &abort_s);
                    if (!ok) break;
                    tc_fence_after();
                    issue_product(tmem + bsel * acc_stride, k_tile, q_blks + bsel * blk_bytes, N, a.bf16, smem_u32(&mma_bar[bsel]));
                    if (it + 2 < n_it) {
                        ok = mbar_wait(smem_u32(&mma_bar[bsel]), use & 1, &abort_s);
                        if (ok) load_q(it + 2);
                    }
                }
                if (!ok) {
                    abort_s = 1;
                    atomicExch(a.status, 1u);
                }
            }
            __syncwarp();
        } else {
            // The log-sum-exps of this warp's half of a block (G * HB <= 128 values) are fetched one block ahead into
            // registers, parked in a per-warp shared-memory row after the current block's arithmetic, and read back as
            // broadcast vector loads: their latency stays off the dependent chain of the statistics.
            float *lw = &lse_w[warp][0][0];
            const int n_ls = G * HB;
            auto fetch = [&](int it, float (&pre)[4]) {
                const int r_base = (rb_first + it) * RB + half * HB;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int n = lane + 32 * k;
                    pre[k] = -kMasked;                                  // past Tq: probability 0
                    if (n < n_ls && it < n_it) {
                        const int g = n / HB, rr = r_base + n % HB;
                        if (rr < a.Tq) pre[k] = __ldg(lse_b + (size_t)g * a.Tq + rr);
                    }
                }
            };
            auto park = [&](int it, const float (&pre)[4]) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int n = lane + 32 * k;
                    if (n < n_ls) lw[(it & 1) * 128 + n] = pre[k];
                }
            };
            float pre[4];
            fetch(0, pre);
            park(0, pre);
            __syncwarp();
            for (int it = 0; it < n_it; ++it) {
                bool ok = mbar_wait(smem_u32(&mma_bar[it & 1]), (unsigned)((it >> 1) & 1), &abort_s);
                ok = __all_sync(0xffffffffu, ok);    // the tensor-memory loads are warp-wide instructions
                if (!ok) {
                    abort_s = 1;
                    atomicExch(a.status, 1u);
                    break;
                }
                fetch(it + 1, pre);
                tc_fence_after();
                const float *lsb = lw + (it & 1) * 128;
                epilogue(it, [&](int g, int, float (&lg)[HB]) {
#pragma unroll
                    for (int i4 = 0; i4 < HB / 4; ++i4) {
                        const float4 f = *reinterpret_cast<const float4 *>(lsb + g * HB + 4 * i4);
                        lg[4 * i4] = f.x; lg[4 * i4 + 1] = f.y; lg[4 * i4 + 2] = f.z; lg[4 * i4 + 3] = f.w;
                    }
                });
                tc_fence_before();
                park(it + 1, pre);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&free_bar[it & 1]));
            }
        }
    } else {
        stage_rows(k_tile, 16, tid, Kb, [&](int row_) { return j0 + row_ < a.Tkv ? Kb + (size_t)(j0 + row_) * kD * esz : nullptr; });
        auto stage_q = [&](int it) {
            if (it < n_it) {
                const int rb = rb_first + it;
                // row n = g * RB + rr of the block is query rb * RB + rr of head g
                stage_rows(q_blks + (it & 1) * blk_bytes, N / 8, tid, Qb, [&](int row_) {
                    const int g = row_ / RB, rr = rb * RB + row_ % RB;
                    return rr < a.Tq ? Qb + ((size_t)g * a.Tq + rr) * kD * esz : nullptr;
                });
                float *ls = lse_s + (it & 3) * N;
                for (int n = tid; n < N; n += kWThreads) {
                    const int g = n / RB, rr = rb * RB + n % RB;
                    ls[n] = rr < a.Tq ? lse_b[(size_t)g * a.Tq + rr] : -kMasked;   // past Tq: probability 0
                }
            }
            cp_async_commit();
        };
        auto issue = [&](int it) {   // warp 0, converged
            tc_fence_after();
            if (elect_one()) issue_product(tmem + (it & 1) * acc_stride, k_tile, q_blks + (it & 1) * blk_bytes, N, a.bf16, smem_u32(&mma_bar[it & 1]));
            __syncwarp();
        };
        stage_q(0);
        stage_q(1);
        cp_async_wait<1>();
        proxy_fence();
        __syncthreads();
        if (warp == 0 && n_it > 0) issue(0);
        bool dead = false;
        for (int it = 0; it < n_it; ++it) {
            // two products in flight, as in pass 1: block it + 1 is issued before block `it` is awaited
            cp_async_wait<0>();
            proxy_fence();
            tc_fence_before();
            __syncthreads();
            dead = dead || abort_s != 0;
            if (warp == 0 && !dead && it + 1 < n_it) issue(it + 1);
            if (!dead && !mbar_wait(smem_u32(&mma_bar[it & 1]), (unsigned)((it >> 1) & 1), &abort_s)) {
                dead = true;
                abort_s = 1;
                atomicExch(a.status, 1u);
            }
            stage_q(it + 2);                        // product `it` is complete: its query buffer is free
            dead = __any_sync(0xffffffffu, dead);   // the tensor-memory loads below are warp-wide instructions
            tc_fence_after();
            if (!dead) {
                const float *lsb = lse_s + (it & 3) * N + half * HB;
                epilogue(it, [&](int g, int, float (&lg)[HB]) {
#pragma unroll
                    for (int i4 = 0; i4 < HB / 4; ++i4) {
                        const float4 f = *reinterpret_cast<const float4 *>(lsb + g * RB + 4 * i4);
                        lg[4 * i4] = f.x; lg[4 * i4 + 1] = f.y; lg[4 * i4 + 2] = f.z; lg[4 * i4 + 3] = f.w;
                    }
                });
            }
        }
        cp_async_wait<0>();
    }
    if (warp < kWorkWarps && half == 1) { part_s[0][row] = s_sum; part_s[1][row] = s_max; part_s[2][row] = s_sq; }
    __syncthreads();
    if (warp < kWorkWarps && half == 0 && j < a.Tkv) {
        const size_t o = (size_t)bh * a.Tkv + j;
        a.sum_attn[o] = s_sum + part_s[0][row];
        a.max_attn[o] = fmaxf(s_max, part_s[1][row]);
        a.sum_sq[o] = s_sq + part_s[2][row];
    }
    tmem_free(tmem, tmem_cols, warp);
}

int pick_rb(int G) { return 32 * G <= 256 ? 32 : 16; }

size_t lse_bytes(int B, int H, int G, int Tq) { return (((size_t)B * H * G * Tq * sizeof(float)) + 255) & ~(size_t)255; }

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link the driver directly)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        cudaGetLastError();
    }
    return fn;
}

// Row-major [heads][T][128] 16-bit tensor as (128 coordinates, T rows, heads); a box (64, box_rows, box_heads) lands
// in shared memory as box_heads * box_rows rows of 128 bytes with the 128-byte swizzle.
bool make_map(CUtensorMap *map, const void *base, int bf16, long long heads, int T, int box_rows, int box_heads) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {128, (cuuint64_t)T, (cuuint64_t)heads};
    const cuuint64_t strides[2] = {256, (cuuint64_t)T * 256};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_heads};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides,
              box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool g_force_thread_copies = false;
int g_last_path = -1;   // 1: tiles arrived by tensor copies, 0: copied by the threads, -1: no call yet

template <class Kern>
cudaError_t allow_smem(Kern kern, int bytes) { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); }

}  // namespace

}  // namespace odmkv

using namespace odmkv;

extern "C" {

size_t odmkv_window_stats_workspace_bytes(int B, int H, int G, int Tq) {
    if (B <= 0 || H <= 0 || G <= 0 || Tq <= 0) return 0;
    return lse_bytes(B, H, G, Tq) + 256;
}

size_t odmkv_window_stats_status_offset(int B, int H, int G, int Tq) { return lse_bytes(B, H, G, Tq); }

int odmkv_window_stats_last_path(void) { return g_last_path; }

void odmkv_window_stats_force_thread_copies(int on) { g_force_thread_copies = on != 0; }

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
    const int smem2 = kTileBytes + 2 * N * kD * 2 + 4 * N * (int)sizeof(float);
    // tensor copies whenever the driver's encoder is there (and not switched off for a test of the other path)
    WinMaps maps;
    memset(&maps, 0, sizeof(maps));
    const bool tma = !g_force_thread_copies && make_map(&maps.q_tile, Q, a.bf16, (long long)B * H * G, Tq, kWRows, 1) &&
                     make_map(&maps.q_blk, Q, a.bf16, (long long)B * H * G, Tq, a.RB, G) &&
                     make_map(&maps.k_tile, K, a.bf16, (long long)B * H, Tkv, kWRows, 1);
    g_last_path = tma ? 1 : 0;
    const dim3 grid1((Tq + kWRows - 1) / kWRows, B * H * G), grid2((Tkv + kWRows - 1) / kWRows, B * H);
    timing_begin("window_lse", st);
    if (tma) {
        if ((e = allow_smem(win_lse_kernel<true>, smem1)) != cudaSuccess) return (int)e;
        win_lse_kernel<true><<<grid1, kTmaThreads, smem1, st>>>(a, maps);
    } else {
        if ((e = allow_smem(win_lse_kernel<false>, smem1)) != cudaSuccess) return (int)e;
        win_lse_kernel<false><<<grid1, kWThreads, smem1, st>>>(a, maps);
    }
    timing_end(st);
    timing_begin("window_cols", st);
    if (a.RB == 32 && tma) {
        if ((e = allow_smem(win_cols_kernel<32, true>, smem2)) != cudaSuccess) return (int)e;
        win_cols_kernel<32, true><<<grid2, kTmaThreads, smem2, st>>>(a, maps);
    } else if (a.RB == 32) {
        if ((e = allow_smem(win_cols_kernel<32, false>, smem2)) != cudaSuccess) return (int)e;
        win_cols_kernel<32, false><<<grid2, kWThreads, smem2, st>>>(a, maps);
    } else if (tma) {
        if ((e = allow_smem(win_cols_kernel<16, true>, smem2)) != cudaSuccess) return (int)e;
        win_cols_kernel<16, true><<<grid2, kTmaThreads, smem2, st>>>(a, maps);
    } else {
        if ((e = allow_smem(win_cols_kernel<16, false>, smem2)) != cudaSuccess) return (int)e;
        win_cols_kernel<16, false><<<grid2, kWThreads, smem2, st>>>(a, maps);
    }
    timing_end(st);
    return launch_status();
}

}  // extern "C"
