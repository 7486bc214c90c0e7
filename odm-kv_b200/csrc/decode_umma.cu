// Decode attention over the 2- and 3-bit banks on the fifth-generation tensor cores (sm_100a:
// tcgen05.mma with the A operand in tensor memory, bulk asynchronous copies for the bank tiles).
//
// Same contract as decode.cu: it replaces the q_len = 1 attention call behind the reference's wrapper
// (kvquant/attention_patch.py:30-55) over the dequantised cache of kvquant/tq_adaptive_backend.py:205-242.
//
// Idea.  A Lloyd-Max codebook for a symmetric density is antisymmetric (c[2^b - 1 - i] = -c[i]), so as a
// function of the b code bits, written as signs x = 2 bit - 1, it only has odd-degree terms:
//     2 bits:  c = A x1 + B x0                                  (exactly two terms)
//     3 bits:  c = A x2 + B x1 + C x0 + D x2 x1 x0              (x2 x1 x0 = sign of the XOR of the three bits)
// A dot product of a query with a decoded key is therefore a sum of dot products of the query with BIT PLANES,
//     q . c[code] = sum_planes w_e (q . bit_e) + const * sum(q),        w_e = 2 coef_e, const = -sum_e coef_e,
// and the same holds for the value side.  A bit plane needs no table: a single AND with 0x01010101 << k turns
// one 32-bit word of a plane into four bytes of an unsigned 8-bit matrix row (value 2^k * bit).  Those bytes are
// the A operand of an integer tensor-core product whose B operand carries the other factor (rotated query or
// softmax weight) as four 8-bit limbs per head, pre-shifted by 7 - k so that every bit position weighs the same.
// The integer product is exact; limbs are recombined in fp32.
//
// Mapping.  A CTA runs two independent pipelines.  Pipeline w owns the slice [w, w + 1) / n_workers of every
// (sample, KV head) unit laid end to end, like a split-K CTA, and streams its tiles of 128 tokens through a ring of
// shared-memory stages filled by one-dimensional bulk copies (TMA, mbarrier transaction counts).  Its warps have
// fixed roles that meet only through mbarriers, so the stages of consecutive tiles overlap:
//   key stagers (4 warps, thread = token): plane words -> 64 registers -> tcgen05.st -> A (128 tokens x 256 plane
//       bits) in tensor memory;
//   value stagers (4 warps, thread = coordinate): the value bank stores planes transposed (bits of a word =
//       tokens), so the same extraction gives A (128 coordinates x 256 (token, plane) bits);
//   issuer (one elected lane): S = A_keys . query limbs (B in shared memory, K-major, s8) into one of two
//       accumulator buffers, and, one tile behind, O^T = A_values . weight limbs (B = the softmax warps' output,
//       MN-major, u8); tcgen05.commit signals the consumers;
//   softmax warps (4 warps): tcgen05.ld of S, logits of the thread's token for every head, running maximum per head
//       (tile maximum exchanged through shared memory), weights W = 2^(z - M) <= 1 written as u32 = four u8 limbs
//       per head; then tcgen05.ld of the previous tile's O^T, whose limbs are recombined and added to the
//       thread's coordinate of the accumulators (one fp32 register per head);
//   producer (one lane): bulk copies, a ring ahead.
// 8-bit, 4-bit, exact and tail tokens go through the CUDA-core kernel of decode.cu; one merge kernel combines all
// partials.  Every wait is bounded; an expired wait marks the pipeline as aborted (it keeps the control flow so
// that no barrier is left waiting) and sets the status word of the workspace.
#include "decode_shared.cuh"

namespace odmkv {

constexpr int kPipes = 2;                      // pipelines per CTA
constexpr int kPipeWarps = 12;                 // key stagers 0-3, value stagers 4-7, softmax 8-11
constexpr int kCtrlWarp0 = kPipes * kPipeWarps;            // issuer warps: kCtrlWarp0 + pipe
constexpr int kProdWarp0 = kCtrlWarp0 + kPipes;            // producer warps: kProdWarp0 + pipe
constexpr int kUmmaThreads = 32 * (kProdWarp0 + kPipes);   // 28 warps
constexpr int kSegBarThreads = 32 * (kPipeWarps + 1);      // the twelve role warps and the issuer warp
constexpr int kTileSlots = kPlaneTile;         // 128 tokens per tile
constexpr int kTmemCols = 512;
constexpr int kPipeCols = 256;                 // per pipeline: A keys [0, 64), A values [64, 128), S at 128 + 32 buf, O^T at 192 + 32 buf
constexpr int kColAK = 0, kColAV = 64, kColDK = 128, kColDV = 192;
constexpr unsigned kUmmaPolls = 1u << 12;       // polls per wait; each may suspend the thread for up to kSuspendNs
constexpr unsigned kSuspendNs = 1000000u;
constexpr float kNegBig = -1.0e30f;
constexpr int kMaxTcClass = 2;                 // classes 1 (2-bit) and 2 (3-bit) take this kernel
constexpr int kSlotBytes = 3 * 4096 + 1024;    // largest tile: 3-bit keys + values (2 x 6144) + two norm rows
constexpr int kStages = 4;

// barrier slots of a pipeline
enum : int { kBarRF = 0, kBarRE = kStages, kBarAKF = 2 * kStages, kBarAKE, kBarAVF, kBarAVE, kBarDKF, kBarDKE = kBarDKF + 2,
             kBarDVF = kBarDKE + 2, kBarDVE = kBarDVF + 2, kBarPF = kBarDVE + 2, kNumBars = kBarPF + 2 };

__host__ __device__ constexpr int umma_bk_bytes(int NT) { return 2 * 256 * 16 * NT; }    // two chunks (3-bit) of 256 plane bits x N bytes
__host__ __device__ constexpr int umma_p_bytes(int NT) { return 2 * 256 * 16 * NT; }     // one tile: up to four planes x 128 tokens x N bytes
__host__ __device__ constexpr int umma_pipe_bytes(int NT) {
    return kStages * kSlotBytes + umma_bk_bytes(NT) + 2 * umma_p_bytes(NT) + 1024;
}
__host__ __device__ constexpr int umma_smem_bytes(int NT) { return kPipes * umma_pipe_bytes(NT) + 1024; }

struct UmmaArgs {
    const float *qrot;
    const float *codebooks;
    float *part_ml;
    float *part_acc;
    unsigned *status;
    int B, H, G, n_workers, slot_base, nslots;
    float scale_log2;
};

// ---- small PTX wrappers ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void named_bar(int id, int nthreads) { asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(nthreads) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// D (tensor memory) (+)= A (tensor memory, u8, row = lane, 32 bytes of K in 8 columns) . B (shared memory, 8-bit)
__device__ __forceinline__ void umma_i8(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d), "r"(a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

// shared-memory matrix descriptor, no swizzle: start address, leading and stride byte offsets (16-byte units)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
           (1ull << 46);
}
// instruction descriptor: s32 accumulator, A u8 K-major (tensor memory), B s8 K-major (keys) or u8 MN-major (values)
__host__ __device__ constexpr uint32_t idesc_i8(int N, bool b_signed, bool b_mn_major) {
    return (2u << 4) | ((b_signed ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ bool mbar_poll(uint32_t bar, unsigned parity) {
    uint32_t ok;
#ifdef ODMKV_NO_SUSPEND_HINT
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
#else
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(kSuspendNs) : "memory");
#endif
    return ok != 0;
}

// bounded wait; an expired wait marks the worker as aborted: later waits return at once, the tensor-core and copy
// issues are skipped, the control flow (and with it every barrier) stays the same
__device__ __forceinline__ void mbar_wait_or_abort(uint32_t bar, unsigned parity, volatile int *abort_flag, unsigned *status) {
    if (*abort_flag) return;
    for (unsigned it = 0; it < kUmmaPolls; ++it)
        if (mbar_poll(bar, parity)) return;
    *abort_flag = 1;
    atomicExch(status, 1u);
}

// one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred P1;\nelect.sync _|P1, 0xffffffff;\nselp.u32 %0, 1, 0, P1;\n}\n" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ int fkey(float x) { const int i = __float_as_int(x); return i ^ ((i >> 31) & 0x7FFFFFFF); }
__device__ __forceinline__ float fkey_inv(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7FFFFFFF)); }
__device__ __forceinline__ float warp_max_f(float x) {
    int k = fkey(x), r;
    asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;\n" : "=r"(r) : "r"(k));
    return fkey_inv(r);
}
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// ---- bit planes --------------------------------------------------------------------------------------------------
// Effective planes of a B-bit level: the B stored planes, then the XORs that carry the odd-degree terms.
template <int B> struct Planes;
template <> struct Planes<2> { static constexpr int kEff = 2; };
template <> struct Planes<3> { static constexpr int kEff = 4; };

// words of effective plane e of one row (16 bytes per stored plane, planes kPlaneTile * 16 bytes apart)
template <int B>
__device__ __forceinline__ uint4 load_eplane(const uint8_t *row0, int e) {
    constexpr int kStride = kTileSlots * 16;
    if (e < B) return *reinterpret_cast<const uint4 *>(row0 + e * kStride);
    const uint4 a = *reinterpret_cast<const uint4 *>(row0), b = *reinterpret_cast<const uint4 *>(row0 + kStride),
                c = *reinterpret_cast<const uint4 *>(row0 + 2 * kStride);
    return make_uint4(a.x ^ b.x ^ c.x, a.y ^ b.y ^ c.y, a.z ^ b.z ^ c.z, a.w ^ b.w ^ c.w);
}

// one plane (4 words) -> 32 matrix-row registers: register 8 wi + k holds bit 8 b + k of word wi in byte b
__device__ __forceinline__ void plane_to_tmem(uint32_t taddr, const uint4 w) {
    uint32_t r[32];
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int wi = 0; wi < 4; ++wi)
#pragma unroll
        for (int k = 0; k < 8; ++k) r[8 * wi + k] = ww[wi] & (0x01010101u << k);
    tmem_st32(taddr, r);
}

// plane coefficients from a codebook: coef_S = 2^-b sum_c cb[c] prod_{i in S} x_i(c); w_e = 2 coef_e, c0 = -sum coef_e
template <int B>
__device__ inline void plane_coefs(const float *cb, float (&w)[Planes<B>::kEff], float &c0) {
    constexpr int n = 1 << B, E = Planes<B>::kEff;
    float coef[E];
#pragma unroll
    for (int e = 0; e < E; ++e) coef[e] = 0.f;
    for (int c = 0; c < n; ++c) {
        const float v = cb[c];
        int par = 0;
#pragma unroll
        for (int e = 0; e < B; ++e) {
            const int bit = (c >> e) & 1;
            par ^= bit;
            coef[e] += bit ? v : -v;
        }
        if (E > B) coef[B] += par ? v : -v;
    }
    c0 = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        coef[e] *= 1.0f / n;
        w[e] = 2.f * coef[e];
        c0 -= coef[e];
    }
}

struct LevelCoefs { float w[4]; float c0; float wmax; };

// ---- per-pipeline shared memory -----------------------------------------------------------------------------------
template <int NT>
struct PipeSmem {
    uint8_t *ring;      // kStages x kSlotBytes
    uint8_t *bk;        // key-side B operand: per chunk 8 steps x [2 K halves][N / 8 row groups][8 rows][16 bytes]
    uint8_t *pbuf;      // value-side B operand, two tiles: per chunk 8 steps x [4 K groups][N / 16 column groups][8 rows][16 bytes]
    float *xch;         // [2][4 warps][8]: per-warp maxima / sums of the softmax warps
    float *hq;          // [2][8]: per head: integer product -> plane sum factor, c0 * sum(q')
    uint64_t *bars;     // kNumBars
    volatile int *abort_flag;
};

template <int NT>
__device__ inline PipeSmem<NT> pipe_smem(uint8_t *base, int pipe) {
    uint8_t *p = base + (size_t)pipe * umma_pipe_bytes(NT);
    PipeSmem<NT> s;
    s.ring = p; p += kStages * kSlotBytes;
    s.bk = p; p += umma_bk_bytes(NT);
    s.pbuf = p; p += 2 * umma_p_bytes(NT);
    s.xch = reinterpret_cast<float *>(p); p += 256;
    s.hq = reinterpret_cast<float *>(p); p += 128;
    s.bars = reinterpret_cast<uint64_t *>(p); p += 8 * kNumBars;
    s.abort_flag = reinterpret_cast<volatile int *>(p);
    return s;
}
static_assert(256 + 128 + 8 * kNumBars + 16 <= 1024, "small area of a pipeline");

// ---- tile sequence of a pipeline ------------------------------------------------------------------------------------
// Pipeline w owns [w * BH, (w + 1) * BH) of the line of BH units, each n_workers long: the fraction [r0, r1) / n_workers
// of every segment of each unit it overlaps.  Order inside a unit: level-major (all chunks of the 2-bit level, then the
// 3-bit level), tiles ascending.  The producer (bulk copies) and every role walk the same sequence.
struct TileSeq {
    long long pos, end;
    int bh, r0, r1, c, ci, t, t_hi, s0, cnt;
    bool in_unit;
    __device__ void init(int w, int BH) { pos = (long long)w * BH; end = pos + BH; in_unit = false; }
    __device__ bool next_unit(int n) {
        if (pos >= end) return false;
        bh = (int)(pos / n); r0 = (int)(pos % n);
        const long long rem = end - pos;
        r1 = (long long)r0 + rem < (long long)n ? (int)(r0 + rem) : n;
        pos += r1 - r0;
        return true;
    }
    __device__ void open_run(const DecodeChunks &chunks, int BH, int n, int c_, int ci_) {
        c = c_; ci = ci_;
        const odmkv_chunk &ch = chunks.ch[ci];
        cnt = ch.seg_count[c * BH + bh];
        const int ntiles = (cnt + kTileSlots - 1) / kTileSlots;
        t = (int)((long long)ntiles * r0 / n);
        t_hi = (int)((long long)ntiles * r1 / n);
        s0 = ch.seg_start[c * BH + bh];
    }
    // tiles of level c_ of the current unit, over all chunks
    __device__ int level_tiles(const DecodeChunks &chunks, int BH, int n, int c_) const {
        int total = 0;
        for (int i = 0; i < chunks.n; ++i) {
            const int ntiles = (chunks.ch[i].seg_count[c_ * BH + bh] + kTileSlots - 1) / kTileSlots;
            total += (int)((long long)ntiles * r1 / n) - (int)((long long)ntiles * r0 / n);
        }
        return total;
    }
    // producer view: next tile in sequence order, or false at the end
    __device__ bool next_tile(const DecodeChunks &chunks, int BH, int n, int &cls, int &chunk_i, int &slot0) {
        for (;;) {
            if (!in_unit) {
                if (!next_unit(n)) return false;
                in_unit = true;
                c = 1; ci = -1; t = 0; t_hi = 0;
            }
            if (t < t_hi) { cls = c; chunk_i = ci; slot0 = s0 + t * kTileSlots; ++t; return true; }
            ++ci;
            if (ci >= chunks.n) { ci = 0; ++c; }
            if (c > kMaxTcClass || chunks.n == 0) { in_unit = false; continue; }
            open_run(chunks, BH, n, c, ci);
        }
    }
};

__device__ inline void issue_tile(const DecodeChunks &chunks, int cls, int chunk_i, int slot0, uint8_t *slot_smem, uint64_t *bar) {
    const odmkv_chunk &ch = chunks.ch[chunk_i];
    const int li = cls - 1, b = cls + 1;   // class 1 -> 2 bits, class 2 -> 3 bits
    const uint32_t code_bytes = (uint32_t)b * 2048u;
    const uint32_t total = 2 * code_bytes + 1024u;
    const uint32_t bar_a = smem_addr(bar), dst = smem_addr(slot_smem);
    const size_t tile = (size_t)slot0 / kTileSlots;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_a), "r"(total) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(ch.k_codes[li] + tile * code_bytes), "r"(code_bytes), "r"(bar_a) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst + code_bytes), "l"(ch.v_codes[li] + tile * code_bytes), "r"(code_bytes), "r"(bar_a) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst + 2 * code_bytes), "l"(ch.k_norm[li] + slot0), "n"(512), "r"(bar_a) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst + 2 * code_bytes + 512), "l"(ch.v_norm[li] + slot0), "n"(512), "r"(bar_a) : "memory");
}

// Everything a role needs to wait: the pipeline's abort flag and the status word
struct Waiter {
    volatile int *abort_flag;
    unsigned *status;
#ifdef ODMKV_PROFILE
    long long *prof;
    __device__ __forceinline__ void wait(uint32_t bar, unsigned parity, int cat = 6) const {
        const long long t0 = clock64();
        mbar_wait_or_abort(bar, parity, abort_flag, status);
        prof[cat] += clock64() - t0;
    }
#else
    __device__ __forceinline__ void wait(uint32_t bar, unsigned parity, int = 0) const { mbar_wait_or_abort(bar, parity, abort_flag, status); }
#endif
    __device__ __forceinline__ bool aborted() const { return *abort_flag != 0; }
};

// ---- key-side B operand of one (unit, level): query limbs (softmax warps, tw = 0..127) ------------------------------
// For plane bit kk of chunk cc (word jw = kk / 32, bit position k = (kk % 32) / 4, byte b = kk % 4): effective plane
// e = 2 cc + jw / 4, coordinate i = 32 (jw % 4) + 8 b + k.  Row n = 4 h + limb holds the balanced base-256 digits of
// round(q'[h][i] * w_e * S_h) << (7 - k), so that sum_kk A[kk] B[n][kk] = 128 * sum bit * round(...) exactly.
template <int B, int NT>
__device__ inline void build_bk(const PipeSmem<NT> &sm, const float *__restrict__ qrot, int bh, int G, const LevelCoefs &lc, int tw, int bar_id) {
    constexpr int N = 16 * NT, E = Planes<B>::kEff, NH = 4 * NT;
    const int warp = tw >> 5, lane = tw & 31;
    // per head: max |q'| and sum q' (thread = coordinate)
    float qv[NH];
#pragma unroll
    for (int h = 0; h < NH; ++h) qv[h] = h < G ? qrot[((size_t)bh * G + h) * kD + tw] : 0.f;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        const float m = warp_max_f(fabsf(qv[h]));
        float s = qv[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) { sm.xch[warp * 8 + h] = m; sm.xch[32 + warp * 8 + h] = s; }
    }
    named_bar(bar_id, 128);
    float S[NH];
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        const float m = fmaxf(fmaxf(sm.xch[h], sm.xch[8 + h]), fmaxf(sm.xch[16 + h], sm.xch[24 + h]));
        const float sum = (sm.xch[32 + h] + sm.xch[40 + h]) + (sm.xch[48 + h] + sm.xch[56 + h]);
        const float den = m * lc.wmax;
        S[h] = den > 0.f ? 4194303.0f / den : 0.f;                       // |round(q' w S)| < 2^22
        if (tw == 0) {
            sm.hq[h] = den > 0.f ? den / (4194303.0f * 128.0f) : 0.f;    // integer product -> sum_planes w_e (q' . bit_e)
            sm.hq[8 + h] = lc.c0 * sum;
        }
    }
    // thread tw fills plane bits tw, tw + 128, ... of every chunk
    for (int kx = tw; kx < E * 128; kx += 128) {
        const int cc = kx >> 8, kk = kx & 255, jw = kk >> 5, k = (kk & 31) >> 2, b = kk & 3;
        const int e = 2 * cc + (jw >> 2), i = 32 * (jw & 3) + 8 * b + k;
        const float we = lc.w[e];
        uint8_t *base = sm.bk + cc * (256 * N) + jw * (32 * N) + ((kk & 31) >> 4) * (N / 8) * 128 + (kk & 15);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            const float q = h < G ? qrot[((size_t)bh * G + h) * kD + i] : 0.f;
            int T = __float2int_rn(q * we * S[h]) << (7 - k);
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                const int n = 4 * h + l;
                const int d = l < 3 ? (int)(int8_t)(T & 0xFF) : T;
                base[(n >> 3) * 128 + (n & 7) * 16] = (uint8_t)d;
                T = (T - d) >> 8;
            }
        }
    }
    proxy_fence();
}

// sum over the 128 softmax threads of up to NH values per thread (result valid in every thread)
template <int NH>
__device__ inline void sm_sum(float (&v)[NH], float *xch, int tw, int bar_id) {
    const int warp = tw >> 5, lane = tw & 31;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        float s = v[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) xch[warp * 8 + h] = s;
    }
    named_bar(bar_id, 128);
#pragma unroll
    for (int h = 0; h < NH; ++h) v[h] = (xch[h] + xch[8 + h]) + (xch[16 + h] + xch[24 + h]);
    named_bar(bar_id, 128);
}

template <int NT>
struct SoftmaxState {
    static constexpr int NH = 4 * NT;
    float M[NH];     // running maximum (log2 domain, includes log2 of the value norm); identical in every softmax thread
    float l[NH];     // this thread's share of the denominators (token role)
    float lw[NH];    // this thread's share of sum W of the current level (token role): the constant term of the value planes
    float O[NH];     // this thread's coordinate of the code-space accumulators (coordinate role)
};

// ---- stagers: one tile of a B-bit level, keys (thread = token) or values (thread = coordinate) ------------------------
// `group` counts the (tile, chunk) products of this side since the kernel started; the A region is free again once
// product group - 1 has completed (bar_empty), and bar_full collects the four stager warps.
template <int B>
__device__ __forceinline__ void stage_tile(const uint8_t *planes, int tw, uint32_t tmem_a, uint32_t bar_empty, uint32_t bar_full,
                                           uint32_t bar_slot, unsigned &group, const Waiter &wt) {
    constexpr int NCH = Planes<B>::kEff / 2;
    const uint8_t *row = planes + tw * 16;
#pragma unroll
    for (int cc = 0; cc < NCH; ++cc) {
        const uint4 w0 = load_eplane<B>(row, 2 * cc), w1 = load_eplane<B>(row, 2 * cc + 1);
        if (group > 0) wt.wait(bar_empty, (group - 1) & 1u, 1);
        tc_fence_after();
        plane_to_tmem(tmem_a, w0);
        plane_to_tmem(tmem_a + 32, w1);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if ((tw & 31) == 0) {
            mbar_arrive(bar_full);
            if (cc == NCH - 1) mbar_arrive(bar_slot);   // this warp has read everything it needs from the ring stage
        }
        ++group;
    }
}

template <int NT>
__global__ void __launch_bounds__(kUmmaThreads, 1) decode_umma_kernel(const DecodeChunks chunks, const UmmaArgs a) {
    extern __shared__ __align__(1024) uint8_t dyn[];
    __shared__ uint32_t tmem_base_s;
    __shared__ LevelCoefs coefs_s[2];
    constexpr int NH = 4 * NT, N = 16 * NT;
    constexpr uint32_t kIdescK = idesc_i8(N, true, false), kIdescV = idesc_i8(N, false, true);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // warp-uniform by construction
    const int BH = a.B * a.H, G = a.G, n = a.n_workers;
    // role of this warp
    const int pipe = warp < kCtrlWarp0 ? warp / kPipeWarps : (warp - kCtrlWarp0) % kPipes;
    const int role = warp < kCtrlWarp0 ? (warp % kPipeWarps) / 4 : (warp < kProdWarp0 ? 3 : 4);   // 0 keys, 1 values, 2 softmax, 3 issuer, 4 producer
    const int tw = warp < kCtrlWarp0 ? 32 * (warp & 3) + lane : lane;                              // token / coordinate of a role thread
    const int w = blockIdx.x * kPipes + pipe;
    const PipeSmem<NT> sm = pipe_smem<NT>(dyn, pipe);
#ifdef ODMKV_PROFILE
    long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long prof_t0 = clock64();
    const Waiter wt{sm.abort_flag, a.status, prof};
#else
    const Waiter wt{sm.abort_flag, a.status};
#endif

    if (role == 3 && lane == 0) {
        for (int i = 0; i < kStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(sm.bars + kBarRF + i)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(sm.bars + kBarRE + i)), "n"(kPipeWarps) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;\n" ::"r"(smem_addr(sm.bars + kBarAKF)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(sm.bars + kBarAKE)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;\n" ::"r"(smem_addr(sm.bars + kBarAVF)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(sm.bars + kBarAVE)) : "memory");
        for (int i = 0; i < 2; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(sm.bars + kBarDKF + i)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;\n" ::"r"(smem_addr(sm.bars + kBarDKE + i)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(sm.bars + kBarDVF + i)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;\n" ::"r"(smem_addr(sm.bars + kBarDVE + i)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;\n" ::"r"(smem_addr(sm.bars + kBarPF + i)) : "memory");
        }
        *sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (tid == 0) {
        coefs_s[0].w[2] = coefs_s[0].w[3] = 0.f;
        plane_coefs<2>(a.codebooks, reinterpret_cast<float(&)[2]>(coefs_s[0].w), coefs_s[0].c0);
        coefs_s[0].wmax = fmaxf(coefs_s[0].w[0], coefs_s[0].w[1]);
        plane_coefs<3>(a.codebooks + 256, coefs_s[1].w, coefs_s[1].c0);
        coefs_s[1].wmax = fmaxf(fmaxf(coefs_s[1].w[0], coefs_s[1].w[1]), fmaxf(coefs_s[1].w[2], coefs_s[1].w[3]));
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_s)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_pipe = __shfl_sync(0xffffffffu, tmem_base_s, 0) + pipe * kPipeCols;
    const uint32_t tmem_lane = tmem_pipe + ((uint32_t)((warp & 3) * 32) << 16);
    const int seg_bar = 1 + pipe, sm_bar = 1 + kPipes + pipe;
    const uint32_t bar0 = smem_addr(sm.bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    if (w < n) {
        if (role == 4) {
            // ---- producer: bulk copies, up to kStages tiles ahead of the slowest consumer
            if (lane == 0) {
                TileSeq prod;
                prod.init(w, BH);
                unsigned g = 0;
                int cls, chunk_i, slot0;
                while (prod.next_tile(chunks, BH, n, cls, chunk_i, slot0)) {
                    const int stage = g % kStages;
                    if (g >= kStages) wt.wait(bar(kBarRE + stage), ((g / kStages) - 1) & 1u);
                    if (!wt.aborted()) issue_tile(chunks, cls, chunk_i, slot0, sm.ring + (size_t)stage * kSlotBytes, sm.bars + kBarRF + stage);
                    ++g;
                }
                // copies still in flight after an abort target this CTA's shared memory: give them a bounded chance to land
                if (wt.aborted()) {
                    for (unsigned i = g > (unsigned)kStages ? g - kStages : 0u; i < g; ++i)
                        for (unsigned it = 0; it < kUmmaPolls; ++it)
                            if (mbar_poll(bar(kBarRF + (int)(i % kStages)), (i / kStages) & 1u)) break;
                }
            }
        } else {
            TileSeq seq;
            seq.init(w, BH);
            unsigned g = 0;            // tiles of this pipeline so far (same in every role)
            unsigned kgrp = 0, vgrp = 0;   // (tile, chunk) products so far, keys / values
            SoftmaxState<NT> st;
            while (seq.next_unit(n)) {
                const int bh = seq.bh;
                if (role == 2) {
#pragma unroll
                    for (int h = 0; h < NH; ++h) { st.M[h] = kNegBig; st.l[h] = 0.f; st.lw[h] = 0.f; st.O[h] = 0.f; }
                }
                for (int c = 1; c <= kMaxTcClass; ++c) {
                    const int ntl = seq.level_tiles(chunks, BH, n, c);
                    if (ntl == 0) continue;
                    const LevelCoefs lc = coefs_s[c - 1];
                    const int nch = c == 1 ? 1 : 2;
                    // every product of the previous segment has completed (the softmax warps waited for the last one)
                    named_bar(seg_bar, kSegBarThreads);
                    if (role == 2) {
                        if (c == 1) build_bk<2, NT>(sm, a.qrot, bh, G, lc, tw, sm_bar);
                        else build_bk<3, NT>(sm, a.qrot, bh, G, lc, tw, sm_bar);
                    }
                    named_bar(seg_bar, kSegBarThreads);

                    if (role == 0 || role == 1) {
                        // ---- stagers
                        for (int ci = 0; ci < chunks.n; ++ci) {
                            seq.open_run(chunks, BH, n, c, ci);
                            for (int t = seq.t; t < seq.t_hi; ++t) {
                                const int stage = g % kStages;
                                wt.wait(bar(kBarRF + stage), (g / kStages) & 1u, 0);
                                const uint8_t *slot = sm.ring + (size_t)stage * kSlotBytes;
                                if (role == 0) {
                                    if (c == 1) stage_tile<2>(slot, tw, tmem_lane + kColAK, bar(kBarAKE), bar(kBarAKF), bar(kBarRE + stage), kgrp, wt);
                                    else stage_tile<3>(slot, tw, tmem_lane + kColAK, bar(kBarAKE), bar(kBarAKF), bar(kBarRE + stage), kgrp, wt);
                                } else {
                                    if (c == 1) stage_tile<2>(slot + 2 * 2048, tw, tmem_lane + kColAV, bar(kBarAVE), bar(kBarAVF), bar(kBarRE + stage), vgrp, wt);
                                    else stage_tile<3>(slot + 3 * 2048, tw, tmem_lane + kColAV, bar(kBarAVE), bar(kBarAVF), bar(kBarRE + stage), vgrp, wt);
                                }
                                ++g;
                            }
                        }
                    } else if (role == 3) {
                        // ---- issuer: keys of tile t, then values of tile t - 1
                        const uint64_t desc_k = smem_desc(smem_addr(sm.bk), (N / 8) * 128, 128);
                        const uint64_t desc_v0 = smem_desc(smem_addr(sm.pbuf), (N / 16) * 128, 128);
                        const bool lead = elect_one();
                        for (int t = 0; t <= ntl; ++t) {
                            if (t < ntl) {
                                const unsigned buf = g & 1u;
                                for (int cc = 0; cc < nch; ++cc) {
                                    wt.wait(bar(kBarAKF), kgrp & 1u, 0);
                                    if (cc == 0 && g >= 2) wt.wait(bar(kBarDKE + buf), ((g >> 1) - 1) & 1u, 1);
                                    tc_fence_after();
                                    if (lead && !wt.aborted()) {
#pragma unroll
                                        for (int s = 0; s < 8; ++s)
                                            umma_i8(tmem_pipe + kColDK + 32 * buf, tmem_pipe + kColAK + 8 * s,
                                                    desc_k + (uint64_t)((cc * 256 * N + s * 32 * N) >> 4), kIdescK, (cc | s) ? 1u : 0u);
                                        umma_commit(bar(kBarAKE));
                                        if (cc == nch - 1) umma_commit(bar(kBarDKF + buf));
                                    }
                                    __syncwarp();
                                    ++kgrp;
                                }
                                ++g;
                            }
                            if (t > 0) {
                                const unsigned gv = g - (t < ntl ? 2u : 1u);   // global index of tile t - 1
                                const unsigned buf = gv & 1u;
                                wt.wait(bar(kBarPF + buf), (gv >> 1) & 1u, 2);
                                if (gv >= 2) wt.wait(bar(kBarDVE + buf), ((gv >> 1) - 1) & 1u, 3);
                                for (int cc = 0; cc < nch; ++cc) {
                                    wt.wait(bar(kBarAVF), vgrp & 1u, 4);
                                    tc_fence_after();
                                    if (lead && !wt.aborted()) {
#pragma unroll
                                        for (int s = 0; s < 8; ++s)
                                            umma_i8(tmem_pipe + kColDV + 32 * buf, tmem_pipe + kColAV + 8 * s,
                                                    desc_v0 + (uint64_t)((buf * umma_p_bytes(NT) + cc * 256 * N + s * 32 * N) >> 4), kIdescV, (cc | s) ? 1u : 0u);
                                        umma_commit(bar(kBarAVE));
                                        if (cc == nch - 1) umma_commit(bar(kBarDVF + buf));
                                    }
                                    __syncwarp();
                                    ++vgrp;
                                }
                            }
                        }
                    } else {
                        // ---- softmax warps (role 2): thread = token for S, thread = coordinate for O^T
                        const float os = lc.wmax * (1.0f / 2147483648.0f);
                        const int jk = tw & 7, jb = (tw & 31) >> 3, jw = tw >> 5;   // this token's place in the plane words of the value bank
                        float ps[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) ps[e] = (lc.w[e] / lc.wmax) * (float)(1u << (31 - jk));
                        int t_seg = 0;
                        float corr[NH];
                        for (int ci = 0; ci < chunks.n; ++ci) {
                            seq.open_run(chunks, BH, n, c, ci);
                            for (int t = seq.t; t < seq.t_hi; ++t, ++t_seg) {
                                const int stage = g % kStages;
                                const unsigned buf = g & 1u;
                                const int nvalid = min(kTileSlots, seq.cnt - t * kTileSlots);
                                wt.wait(bar(kBarRF + stage), (g / kStages) & 1u, 0);
                                const uint8_t *slot = sm.ring + (size_t)stage * kSlotBytes;
                                const int bq = c + 1;
                                const float kn = reinterpret_cast<const float *>(slot + 2 * bq * 2048)[tw];
                                const float vn = reinterpret_cast<const float *>(slot + 2 * bq * 2048 + 512)[tw];
                                // ---- logits of this thread's token (log2 domain, plus log2 of the value norm)
                                float z[NH];
                                {
                                    wt.wait(bar(kBarDKF + buf), (g >> 1) & 1u, 1);
                                    tc_fence_after();
                                    uint32_t d[N];
#pragma unroll
                                    for (int c16 = 0; c16 < NT; ++c16)
                                        tmem_ld16(tmem_lane + kColDK + 32 * buf + 16 * c16, reinterpret_cast<uint32_t(&)[16]>(d[16 * c16]));
                                    tmem_ld_wait();
                                    tc_fence_before();
                                    __syncwarp();
                                    if (lane == 0) mbar_arrive(bar(kBarDKE + buf));
                                    const bool valid = tw < nvalid;
                                    const float vnc = fmaxf(vn, 1e-30f);
                                    const float lv = valid ? __log2f(vnc) : kNegBig;
                                    const float kf = kn * a.scale_log2;
#pragma unroll
                                    for (int h = 0; h < NH; ++h) {
                                        const int lo = (int)d[4 * h] + 256 * (int)d[4 * h + 1], hi = (int)d[4 * h + 2] + 256 * (int)d[4 * h + 3];
                                        const float f = fmaf(65536.f, (float)hi, (float)lo);
                                        const float s = fmaf(f, sm.hq[h], sm.hq[8 + h]);
                                        z[h] = valid ? fmaf(s, kf, lv) : kNegBig;
                                    }
                                }
                                // ---- tile maximum per head over the four warps, running-maximum update
#pragma unroll
                                for (int h = 0; h < NH; ++h) {
                                    const float m = warp_max_f(z[h]);
                                    if (lane == 0) sm.xch[(t_seg & 1) * 32 + (warp & 3) * 8 + h] = m;
                                }
#ifdef ODMKV_PROFILE
                                const long long tb0 = clock64();
#endif
                                named_bar(sm_bar, 128);
#ifdef ODMKV_PROFILE
                                prof[3] += clock64() - tb0;
#endif
                                float W[NH];
                                {
                                    const float rv = tw < nvalid ? __fdividef(1.0f, fmaxf(vn, 1e-30f)) : 0.f;
                                    const float *xm = sm.xch + (t_seg & 1) * 32;
#pragma unroll
                                    for (int h = 0; h < NH; ++h) {
                                        const float mt = fmaxf(fmaxf(xm[h], xm[8 + h]), fmaxf(xm[16 + h], xm[24 + h]));
                                        const float mn = fmaxf(st.M[h], mt);
                                        corr[h] = fast_ex2(st.M[h] - mn);   // 1 when unchanged, 0 for the first tile
                                        st.M[h] = mn;
                                        W[h] = fast_ex2(z[h] - mn);         // <= 1; 0 for padding slots
                                        st.l[h] = fmaf(st.l[h], corr[h], W[h] * rv);
                                        st.lw[h] = fmaf(st.lw[h], corr[h], W[h]);
                                    }
                                }
                                // ---- weight rows of this token, every plane of the tile: u32 = four u8 limbs per head
                                // (the buffer is free: the products of tile g - 2 completed before its O^T was read)
                                {
                                    uint8_t *pb = sm.pbuf + buf * umma_p_bytes(NT);
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        if (e < 2 * nch) {
                                            const int kk = 32 * (4 * (e & 1) + jw) + 4 * jk + jb;   // row inside the chunk's B operand
                                            uint8_t *row = pb + (e >> 1) * (256 * N) + (kk >> 5) * (32 * N) + ((kk & 31) >> 3) * (N / 16) * 128 + (kk & 7) * 16;
#pragma unroll
                                            for (int g4 = 0; g4 < NT; ++g4) {
                                                uint4 v;
                                                v.x = __float2uint_rn(W[4 * g4] * ps[e]); v.y = __float2uint_rn(W[4 * g4 + 1] * ps[e]);
                                                v.z = __float2uint_rn(W[4 * g4 + 2] * ps[e]); v.w = __float2uint_rn(W[4 * g4 + 3] * ps[e]);
                                                *reinterpret_cast<uint4 *>(row + g4 * 128) = v;
                                            }
                                        }
                                    }
                                    proxy_fence();
                                    __syncwarp();
                                    if (lane == 0) { mbar_arrive(bar(kBarPF + buf)); mbar_arrive(bar(kBarRE + stage)); }
                                }
                                // ---- O^T of the previous tile (weights relative to the maximum before this tile's update)
                                if (t_seg > 0) {
                                    const unsigned gp = g - 1, pbuf_i = gp & 1u;
                                    wt.wait(bar(kBarDVF + pbuf_i), (gp >> 1) & 1u, 2);
                                    tc_fence_after();
                                    uint32_t d[N];
#pragma unroll
                                    for (int c16 = 0; c16 < NT; ++c16)
                                        tmem_ld16(tmem_lane + kColDV + 32 * pbuf_i + 16 * c16, reinterpret_cast<uint32_t(&)[16]>(d[16 * c16]));
                                    tmem_ld_wait();
                                    tc_fence_before();
                                    __syncwarp();
                                    if (lane == 0) mbar_arrive(bar(kBarDVE + pbuf_i));
#pragma unroll
                                    for (int h = 0; h < NH; ++h) {
                                        const uint32_t lo = d[4 * h] + 256u * d[4 * h + 1], hi = d[4 * h + 2] + 256u * d[4 * h + 3];
                                        st.O[h] = fmaf(fmaf(65536.f, (float)hi, (float)lo), os, st.O[h]);
                                    }
                                }
#pragma unroll
                                for (int h = 0; h < NH; ++h) st.O[h] *= corr[h];
                                ++g;
                            }
                        }
                        // ---- drain: O^T of the segment's last tile, then the constant term of the level's planes
                        {
                            const unsigned gp = g - 1, pbuf_i = gp & 1u;
                            wt.wait(bar(kBarDVF + pbuf_i), (gp >> 1) & 1u, 2);
                            tc_fence_after();
                            uint32_t d[N];
#pragma unroll
                            for (int c16 = 0; c16 < NT; ++c16)
                                tmem_ld16(tmem_lane + kColDV + 32 * pbuf_i + 16 * c16, reinterpret_cast<uint32_t(&)[16]>(d[16 * c16]));
                            tmem_ld_wait();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar(kBarDVE + pbuf_i));
#pragma unroll
                            for (int h = 0; h < NH; ++h) {
                                const uint32_t lo = d[4 * h] + 256u * d[4 * h + 1], hi = d[4 * h + 2] + 256u * d[4 * h + 3];
                                st.O[h] = fmaf(fmaf(65536.f, (float)hi, (float)lo), os, st.O[h]);
                            }
                            float lw[NH];
#pragma unroll
                            for (int h = 0; h < NH; ++h) lw[h] = st.lw[h];
                            sm_sum<NH>(lw, sm.xch, tw, sm_bar);
#pragma unroll
                            for (int h = 0; h < NH; ++h) { st.O[h] = fmaf(lc.c0, lw[h], st.O[h]); st.lw[h] = 0.f; }
                        }
                    }
                }
                // ---- partial of this (pipeline, unit): natural-log maximum, denominator, code-space accumulator
                if (role == 2) {
                    float l[NH];
#pragma unroll
                    for (int h = 0; h < NH; ++h) l[h] = st.l[h];
                    sm_sum<NH>(l, sm.xch, tw, sm_bar);
                    const int GP = round_gp(G);
                    const int slot_i = w - (int)(((long long)bh * n) / BH);
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        if (h < GP) {
                            const size_t pi = ((size_t)bh * a.nslots + a.slot_base + slot_i) * GP + h;
                            a.part_acc[pi * 2 * kD + tw] = h < G ? st.O[h] : 0.f;
                            a.part_acc[pi * 2 * kD + kD + tw] = 0.f;
                            if (tw == 0) {
                                a.part_ml[pi * 2] = (h < G && st.M[h] > kNegBig) ? st.M[h] * 0.6931471805599453f : -INFINITY;
                                a.part_ml[pi * 2 + 1] = h < G ? l[h] : 0.f;
                            }
                        }
                    }
                }
            }
        }
    }
#ifdef ODMKV_PROFILE
    if (blockIdx.x == 7 && pipe == 0 && lane == 0 && (role >= 3 || (warp & 3) == 0)) {
        prof[7] = clock64() - prof_t0;
        for (int i = 0; i < 8; ++i) reinterpret_cast<long long *>(a.status)[2 + role * 8 + i] = prof[i];
    }
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base_s), "r"((uint32_t)kTmemCols) : "memory");
}

static int num_sms_cached() {
    static int table[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (table[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        table[dev] = n;
    }
    return table[dev];
}

// one helper stream and two events per device, created on first use (host objects, no device memory)
struct SideStream { cudaStream_t stream; cudaEvent_t fork, join; bool ok; };
static SideStream *side_stream() {
    static SideStream table[64] = {};
    static bool tried[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!tried[dev]) {
        tried[dev] = true;
        SideStream &s = table[dev];
        s.ok = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) == cudaSuccess &&
               cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) == cudaSuccess &&
               cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) == cudaSuccess;
    }
    return table[dev].ok ? &table[dev] : nullptr;
}

}  // namespace odmkv

using namespace odmkv;

extern "C" {

int odmkv_decode_attn_mma(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                          const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                          const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                          int out_dtype, float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                          void *stream) {
    DecodeChunks dc;
    int rc = decode_check_args(q, q_dtype, chunks, n_chunks, cache_dtype, tail_k, tail_v, tail_len, tail_cap, pi_k, pi_v, codebooks,
                               B, H, G, out, out_dtype, n_splits, workspace, &dc);
    if (rc) return rc;
    // 4-bit / 8-bit / exact / tail tokens: a few CTAs of the CUDA-core kernel per (b, h)
    long long side_tokens = tail_len;
    for (int i = 0; i < n_chunks; ++i)
        side_tokens += ((long long)chunks[i].cap[3] + chunks[i].cap[4] + chunks[i].cap[5]) / ((long long)B * H) + 1;
    int ns_side = (int)((side_tokens + 127) / 128);   // one 32-token group per warp of the CUDA-core kernel
    if (ns_side < 1) ns_side = 1;
    if (ns_side > 8) ns_side = 8;
    const int nslots = n_splits + ns_side;
    DecodeWs ws;
    if (workspace_bytes < decode_ws_layout(B, H, G, nslots, &ws, (unsigned char *)workspace)) return ODMKV_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int BH = B * H;
    cudaMemsetAsync(ws.status, 0, sizeof(unsigned), st);
    timing_begin("decode_rotate", st);
    launch_rotate_q(q, q_dtype, pi_k, ws, BH * G, st);
    timing_end(st);
    {
        SideStream *fk = side_stream();
        if (fk) cudaEventRecord(fk->fork, st);
    }
    UmmaArgs m;
    m.qrot = ws.qrot; m.codebooks = codebooks; m.part_ml = ws.part_ml; m.part_acc = ws.part_acc; m.status = ws.status;
    // workers (pipelines): two per SM, fewer when the cache is short (at least two tiles each) or when the caller's slot
    // count bounds the workers that may overlap one unit
    long long total_tiles = 0;
    for (int i = 0; i < n_chunks; ++i) total_tiles += ((long long)chunks[i].cap[1] + chunks[i].cap[2]) / kPlaneTile;
    long long n_workers = (long long)kPipes * num_sms_cached();
    if (n_workers > total_tiles / 2) n_workers = total_tiles / 2;
    if (n_splits >= 2) {
        if (n_workers > (long long)(n_splits - 1) * BH) n_workers = (long long)(n_splits - 1) * BH;
    } else {
        if (n_workers > BH) n_workers = BH;
        while (n_workers > 1 && BH % n_workers != 0) --n_workers;   // one slot: every unit belongs to exactly one worker
    }
    if (n_workers < 1) n_workers = 1;
    m.B = B; m.H = H; m.G = G; m.n_workers = (int)n_workers; m.slot_base = 0; m.nslots = nslots;
    m.scale_log2 = scale * 1.4426950408889634f;
    dim3 grid((unsigned)((n_workers + kPipes - 1) / kPipes));
    {
        static bool attr_set[64] = {};   // per device: the opt-in only has to happen once
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            cudaError_t e1 = cudaFuncSetAttribute(decode_umma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, umma_smem_bytes(1));
            cudaError_t e2 = cudaFuncSetAttribute(decode_umma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, umma_smem_bytes(2));
            if (e1 != cudaSuccess) return (int)e1;
            if (e2 != cudaSuccess) return (int)e2;
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    timing_begin("decode_main", st);
    if (G <= 4) decode_umma_kernel<1><<<grid, kUmmaThreads, umma_smem_bytes(1), st>>>(dc, m);
    else decode_umma_kernel<2><<<grid, kUmmaThreads, umma_smem_bytes(2), st>>>(dc, m);
    timing_end(st);
    DecodeArgs a;
    a.qrot = ws.qrot; a.qf = ws.qf; a.tail_k = tail_k; a.tail_v = tail_v; a.codebooks = codebooks;
    a.part_ml = ws.part_ml; a.part_acc = ws.part_acc; a.tail_len = tail_len; a.tail_cap = tail_cap;
    a.B = B; a.H = H; a.G = G; a.nsplit = ns_side; a.slot_base = n_splits; a.nslots = nslots;
    a.class_mask = (1 << 3) | (1 << 4) | (1 << 5) | (1 << 6); a.scale = scale;
    // the exact / tail kernel only needs the rotated queries, so it runs beside the tensor-core kernel on a
    // second stream (fork after the rotation, join before the merge)
    SideStream *ss = side_stream();
    if (ss) {
        cudaStreamWaitEvent(ss->stream, ss->fork, 0);
        timing_begin("decode_side", ss->stream);
        launch_decode_cuda_core(dc, a, cache_dtype, ss->stream);
        timing_end(ss->stream);
        cudaEventRecord(ss->join, ss->stream);
        cudaStreamWaitEvent(st, ss->join, 0);
    } else {
        timing_begin("decode_side", st);
        launch_decode_cuda_core(dc, a, cache_dtype, st);
        timing_end(st);
    }
    timing_begin("decode_merge", st);
    launch_decode_merge(ws, pi_v, BH, G, nslots, out, out_dtype, lse, st, n_splits, (int)n_workers);
    timing_end(st);
    return launch_status();
}

}  // extern "C"
