// Tensor-core decode attention over the 2/3/4-bit banks (sm_100a).
//
// Same contract as decode.cu (it replaces the q_len = 1 attention call behind the reference's wrapper,
// kvquant/attention_patch.py:30-55, over the dequantised cache of kvquant/tq_adaptive_backend.py:205-242),
// different machine mapping.  A warp consumes one bank tile of 16 tokens at a time:
//   * the tile's key codes arrive as one 8*b-byte load per lane, already in m16n8k16 A-fragment order;
//     a pair of codes (2*b bits) indexes a per-lane copy of a small table of half2 centroid pairs, so
//     one shared-memory read yields one A register;
//   * S = K_dec (16 x 128) . q'^T (128 x 8) runs as 8 HMMA steps; the 8 columns are the fp16 high and
//     low limbs of the rotated queries of up to 4 heads (two column tiles for up to 8 heads), so the
//     query enters with ~22 bits;
//   * softmax weights use a lazily updated warp-wide running maximum of logit + log2(value norm), which
//     bounds every weight by 2^6 and keeps the fp16 P operand in range whatever the norms are;
//   * P is transposed in registers with movmatrix and O^T (128 x 8) += V_dec^T (128 x 16) . P (16 x 8)
//     runs as 8 more HMMA steps with the value codes decoded through the same tables.
// 8-bit tokens, the exact bank and the dense tail go through the CUDA-core kernel of decode.cu in a
// second launch that writes its own partial slots; one merge kernel combines everything.
#include "decode_shared.cuh"

namespace odmkv {

constexpr int kMmaThreads = 256;
constexpr int kMmaWarps = kMmaThreads / 32;
#ifndef ODMKV_MMA_CTAS
#define ODMKV_MMA_CTAS 2
#endif
#ifndef ODMKV_TILES_PER_ITER
#define ODMKV_TILES_PER_ITER 3
#endif
constexpr float kTau = 6.0f;   // lazy-maximum slack in log2 units: weights stay below 2^6
constexpr float kNegBig = -1.0e30f;   // stands for -inf where a finite value keeps the arithmetic free of special cases

struct MmaArgs {
    const float *qrot;
    const float *codebooks;
    float *part_ml;
    float *part_acc;
    int B, H, G, n_cta, slot_base, nslots;   // n_cta CTAs share the B*H units evenly; nslots = partial slots per unit
    float scale_log2;      // softmax scale * log2(e)
    float lut_scale[3];    // centroids are stored in the tables as fp16(c * lut_scale[li])
};

__device__ inline void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ inline uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

__device__ inline float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// loads from a 32-bit shared-space address (no generic-pointer arithmetic on the lookup path)
__device__ inline uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ inline uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ inline uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ inline uint32_t cvt_f16x2(float lo, float hi) {   // one instruction: two floats -> half2
    uint32_t v;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(v) : "f"(hi), "f"(lo));
    return v;
}

template <int N>
__device__ inline void cp_async(uint32_t s, const void *gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(s), "l"(gmem), "n"(N) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ inline uint32_t pack_half2(__half lo, __half hi) {
    return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

// pair field f (2*B bits at bit 2*B*f) of a little-endian word array; f is a compile-time constant
// at every call site, so the branch and the shifts fold away
template <int B>
__device__ inline uint32_t pair_field(const uint32_t *w, int f) {
    const int off = 2 * B * f, wi = off >> 5, sh = off & 31;
    uint32_t v;
    if (sh + 2 * B <= 32) v = w[wi] >> sh;
    else v = __funnelshift_r(w[wi], w[wi + 1], sh);
    return v & ((1u << (2 * B)) - 1u);
}

// Table lookups.  One shared-memory table serves the 2- and 3-bit levels; row r (256 bytes) holds
//   bytes [0, 128):   for the code byte r (four 2-bit codes): two half2 (low nibble pair, high nibble pair),
//                     16 copies of 8 bytes -- lane l reads copy l % 16, so a half-warp never collides;
//   bytes [128, 256): for r < 64, the 6-bit pair field r of the 3-bit level: one half2, 32 copies.
// With a 256-byte row the table offset of a 2-bit lookup is (code byte << 8) | lane offset, which a
// single byte-permute builds from the data word and a lane constant; the table base is a link-time
// constant folded into the load.  The 4-bit level (one byte per pair) uses a separate single-copy table.
constexpr int kLutRow = 256;
constexpr int kLutBytes = 256 * kLutRow;             // 64 KiB
constexpr int kLut4Bytes = 256 * 4;
constexpr int kStageBytes = kLutBytes + kLut4Bytes;

extern __shared__ __align__(128) uint8_t g_dyn[];   // [kLutBytes combined table][kLut4Bytes]

// 3-bit pair field f of a row part, already shifted to bits 8..13 and merged with the lane offset
__device__ inline uint32_t field3_offset(const uint32_t *w, int f, uint32_t lane_off) {
    const int off = 6 * f, wi = off >> 5, sh = off & 31;
    uint32_t v;
    if (sh < 8) v = w[wi] << (8 - sh);
    else if (sh + 6 <= 32) v = w[wi] >> (sh - 8);
    else v = __funnelshift_r(w[wi], w[wi + 1], sh - 8);
    return (v & 0x3F00u) | lane_off;
}

// Both banks store, for HMMA step j (a key step s or a value block m), the four A registers a0..a3 as
// fields 4j..4j+3, so one routine decodes either.
template <int B>
__device__ inline void decode_step(uint32_t lane_off, const uint32_t *w, int j, uint32_t (&a)[4]) {
    if (B == 2) {
        // bytes 2j, 2j+1 = fields (4j, 4j+1), (4j+2, 4j+3): each 64-bit table entry is an aligned register pair
        const int b0 = 2 * j, b1 = 2 * j + 1;
        const uint2 e0 = *reinterpret_cast<const uint2 *>(g_dyn + __byte_perm(w[b0 >> 2], lane_off, 0x5504 | ((b0 & 3) << 4)));
        const uint2 e1 = *reinterpret_cast<const uint2 *>(g_dyn + __byte_perm(w[b1 >> 2], lane_off, 0x5504 | ((b1 & 3) << 4)));
        a[0] = e0.x; a[1] = e0.y; a[2] = e1.x; a[3] = e1.y;
    } else if (B == 3) {
#pragma unroll
        for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const uint32_t *>(g_dyn + field3_offset(w, 4 * j + r, lane_off));
    } else {
        const uint32_t *t4 = reinterpret_cast<const uint32_t *>(g_dyn + kLutBytes);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int f = 4 * j + r;
            a[r] = t4[__byte_perm(w[f >> 2], 0, 0x4440 | (f & 3))];
        }
    }
}

template <int NT>
struct MmaState {
    float M[2], l[2];        // per head column of this lane (two heads per lane)
    float O[8][4];           // O^T fragments: [16-coordinate block][c0..c3]; NT = 1: columns 4..7 take the low limbs of the weights,
                             // NT = 2: eight heads, weights enter as fp16 (the denominators use the same rounded weights)
};

template <int B>
struct TileRegs {
    uint32_t kw[2 * B], vw[2 * B];
    float kn0, kn1, vn0, vn1;
};

// Consume U (1 or 2) tiles at once.  With two tiles the two dependency chains (table load -> HMMA ->
// softmax -> HMMA) interleave, which is what keeps the schedulers fed at 4 warps each.  qBs holds the
// query B fragments in shared memory as [column tile][step][lane] register pairs.
template <int B, int NT, int U, bool FULL>
__device__ inline void process_tiles(MmaState<NT> &st, const TileRegs<B> (&tr)[U], const int (&nvalid)[U], const uint2 *__restrict__ qBs,
                                     uint32_t lane_off, int lane, float kfac, float inv_lut_scale) {
    const int g = lane >> 2, t = lane & 3;
    // ---- S = K_dec . q'^T
    float S[U][NT][4];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) S[u][nt][i] = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        uint2 qb[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) qb[nt] = qBs[(nt * 8 + s) * 32 + lane];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            uint32_t a[4];
            decode_step<B>(lane_off, tr[u].kw, s, a);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma16816(S[u][nt], a, qb[nt].x, qb[nt].y);
        }
    }
    // ---- logits in the log2 domain plus log2(value norm); rows past the segment's end drop out branch-free
    float z[U][4], rv[U][2];
    float zm0 = kNegBig, zm1 = kNegBig;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        float sv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (NT == 1) sv[i] = S[u][0][i] + __shfl_xor_sync(0xffffffffu, S[u][0][i], 2);   // high + low query limbs
            else sv[i] = S[u][0][i] + S[u][NT - 1][i];
        }
        const bool ok0 = FULL || g < nvalid[u], ok1 = FULL || g + 8 < nvalid[u];
        const float vc0 = fmaxf(tr[u].vn0, 1e-30f) * inv_lut_scale, vc1 = fmaxf(tr[u].vn1, 1e-30f) * inv_lut_scale;
        const float lv0 = ok0 ? __log2f(vc0) : kNegBig, lv1 = ok1 ? __log2f(vc1) : kNegBig;
        rv[u][0] = ok0 ? __fdividef(1.0f, vc0) : 0.f;
        rv[u][1] = ok1 ? __fdividef(1.0f, vc1) : 0.f;
        const float f0 = tr[u].kn0 * kfac, f1 = tr[u].kn1 * kfac;
        z[u][0] = fmaf(sv[0], f0, lv0);
        z[u][1] = fmaf(sv[1], f0, lv0);
        z[u][2] = fmaf(sv[2], f1, lv1);
        z[u][3] = fmaf(sv[3], f1, lv1);
        zm0 = fmaxf(zm0, fmaxf(z[u][0], z[u][2]));
        zm1 = fmaxf(zm1, fmaxf(z[u][1], z[u][3]));
    }
    // ---- lazily updated running maximum (one vote per group of tiles)
    const bool need = (zm0 > st.M[0] + kTau) || (zm1 > st.M[1] + kTau);
    if (__any_sync(0xffffffffu, need)) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            zm0 = fmaxf(zm0, __shfl_xor_sync(0xffffffffu, zm0, o));
            zm1 = fmaxf(zm1, __shfl_xor_sync(0xffffffffu, zm1, o));
        }
        const float n0 = fmaxf(st.M[0], zm0), n1 = fmaxf(st.M[1], zm1);
        const float c0 = fast_exp2(st.M[0] - n0), c1 = fast_exp2(st.M[1] - n1);   // 2^(-1e30 - n) = 0 for the first tile
        st.M[0] = n0; st.M[1] = n1;
        st.l[0] *= c0; st.l[1] *= c1;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            st.O[m][0] *= c0; st.O[m][1] *= c1; st.O[m][2] *= c0; st.O[m][3] *= c1;
        }
    }
    // ---- weights and the P operand (fp16 high and low limb of every weight, two weights per conversion)
    const float m0 = st.M[0], m1 = st.M[1];
    uint32_t pb[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const float W0 = fast_exp2(z[u][0] - m0), W1 = fast_exp2(z[u][1] - m1), W2 = fast_exp2(z[u][2] - m0), W3 = fast_exp2(z[u][3] - m1);
        const uint32_t hi01 = cvt_f16x2(W0, W1), hi23 = cvt_f16x2(W2, W3);
        const float2 b01 = __half22float2(*reinterpret_cast<const __half2 *>(&hi01));
        const float2 b23 = __half22float2(*reinterpret_cast<const __half2 *>(&hi23));
        if (NT == 1) {
            st.l[0] = fmaf(W0, rv[u][0], fmaf(W2, rv[u][1], st.l[0]));
            st.l[1] = fmaf(W1, rv[u][0], fmaf(W3, rv[u][1], st.l[1]));
            const uint32_t lo01 = cvt_f16x2(W0 - b01.x, W1 - b01.y), lo23 = cvt_f16x2(W2 - b23.x, W3 - b23.y);
            const bool low = (t & 2) != 0;   // columns 4..7 carry the low limbs
            pb[u][0] = movmatrix_trans(low ? lo01 : hi01);
            pb[u][1] = movmatrix_trans(low ? lo23 : hi23);
        } else {
            // numerator and denominator see the same fp16-rounded weights
            st.l[0] = fmaf(b01.x, rv[u][0], fmaf(b23.x, rv[u][1], st.l[0]));
            st.l[1] = fmaf(b01.y, rv[u][0], fmaf(b23.y, rv[u][1], st.l[1]));
            pb[u][0] = movmatrix_trans(hi01);
            pb[u][1] = movmatrix_trans(hi23);
        }
    }
    // ---- O^T += V_dec^T . P
#pragma unroll
    for (int m = 0; m < 8; ++m) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            uint32_t a[4];
            decode_step<B>(lane_off, tr[u].vw, m, a);
#pragma unroll
            mma16816(st.O[m], a, pb[u][0], pb[u][1]);
        }
    }
}

// Tile data goes straight from global memory to registers: every lane loads its own key chunk, value
// chunk and four norms (its fragment rows g and g+8), one tile ahead of the tile being consumed, so the
// loads of tile i+1 are in flight while tile i is decoded.  Nothing is staged in shared memory, which is
// left to the lookup tables.
__device__ inline uint4 ldg128(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ inline uint2 ldg64(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

template <int B>
__device__ inline void load_words(const uint8_t *__restrict__ p, uint32_t (&w)[2 * B]) {
    if (B == 2) {
        const uint4 v = ldg128(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if (B == 3) {
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const uint2 v = ldg64(p + 8 * i);
            w[2 * i] = v.x; w[2 * i + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 v = ldg128(p + 16 * i);
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    }
}

template <int B>
struct TilePtrs {   // this lane's addresses inside the current tile of the four arrays
    const uint8_t *k, *v;
    const float *kn, *vn;
    __device__ void advance(int tiles) {
        k += (size_t)tiles * 256 * B; v += (size_t)tiles * 256 * B;
        kn += tiles * 16; vn += tiles * 16;
    }
};

template <int B>
__device__ inline void load_tile(TileRegs<B> &r, const TilePtrs<B> &p) {
    load_words<B>(p.k, r.kw);
    load_words<B>(p.v, r.vw);
    // volatile so that these stay with the tile's other loads, one iteration ahead of their use
    asm volatile("ld.global.nc.f32 %0, [%1];\n" : "=f"(r.kn0) : "l"(p.kn));
    asm volatile("ld.global.nc.f32 %0, [%1+32];\n" : "=f"(r.kn1) : "l"(p.kn));
    asm volatile("ld.global.nc.f32 %0, [%1];\n" : "=f"(r.vn0) : "l"(p.vn));
    asm volatile("ld.global.nc.f32 %0, [%1+32];\n" : "=f"(r.vn1) : "l"(p.vn));
}

template <int B, int NT>
__device__ inline void process_segment(MmaState<NT> &st, const odmkv_chunk &ch, int s0, int cnt, int r0, int r1, int rn, int warp, int lane,
                                       const uint2 *__restrict__ qBs, uint32_t lane_off, float scale_log2, float lut_scale) {
    constexpr int LI = B - 2;
    const int ntiles = (cnt + 15) >> 4;
    const int t_lo = (int)((long long)ntiles * r0 / rn), t_hi = (int)((long long)ntiles * r1 / rn);   // this CTA's share of the tiles
    const float kfac = scale_log2 / lut_scale, inv_ls = 1.0f / lut_scale;
    int ti = t_lo + warp;
    if (ti >= t_hi) return;
    constexpr int stride = kMmaWarps;
    TilePtrs<B> p;
    {
        const size_t tile0 = (size_t)(s0 >> 4) + ti;
        p.k = ch.k_codes[LI] + (tile0 * 32 + lane) * 8 * B;
        p.v = ch.v_codes[LI] + (tile0 * 32 + lane) * 8 * B;
        p.kn = ch.k_norm[LI] + tile0 * 16 + (lane >> 2);
        p.vn = ch.v_norm[LI] + tile0 * 16 + (lane >> 2);
    }
    // this warp's tiles kU at a time (ti, ti + 8, ...); the remainder goes one by one
    constexpr int kU = (B == 2 && NT == 1) ? ODMKV_TILES_PER_ITER : 2;
    for (; ti + (kU - 1) * kMmaWarps < t_hi; ti += kU * kMmaWarps) {
        TileRegs<B> tr[kU];
        int nv[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            load_tile<B>(tr[u], p);
            p.advance(stride);
            nv[u] = cnt - (ti + u * kMmaWarps) * 16;
        }
        if (nv[kU - 1] >= 16) process_tiles<B, NT, kU, true>(st, tr, nv, qBs, lane_off, lane, kfac, inv_ls);
        else process_tiles<B, NT, kU, false>(st, tr, nv, qBs, lane_off, lane, kfac, inv_ls);
    }
    for (; ti < t_hi; ti += kMmaWarps) {
        TileRegs<B> tr[1];
        load_tile<B>(tr[0], p);
        p.advance(stride);
        const int nv[1] = {cnt - ti * 16};
        process_tiles<B, NT, 1, false>(st, tr, nv, qBs, lane_off, lane, kfac, inv_ls);
    }
}

template <int NT>
__global__ void __launch_bounds__(kMmaThreads, ODMKV_MMA_CTAS) decode_mma_kernel(const DecodeChunks chunks, const MmaArgs a) {
    __shared__ float Osh[4 * NT][kD];
    __shared__ float lsh[4 * NT], Msh[4 * NT];
    __shared__ float warpM[kMmaWarps][4 * NT];
    __shared__ uint2 qBs[NT * 8 * 32];   // query B fragments: [column tile][step][lane]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int BH = a.B * a.H, G = a.G;
    constexpr int NH = 4 * NT;   // head slots of this kernel variant

    // ---- tables of half2 centroid pairs (once per CTA)
    {
        const float *c2 = a.codebooks, *c3 = a.codebooks + 256, *c4 = a.codebooks + 512;
        const float s2 = a.lut_scale[0], s3 = a.lut_scale[1], s4 = a.lut_scale[2];
        for (int e = tid; e < 256 * 16; e += kMmaThreads) {
            const int v = e >> 4, c = e & 15;
            uint2 ent;
            ent.x = pack_half2(__float2half_rn(c2[v & 3] * s2), __float2half_rn(c2[(v >> 2) & 3] * s2));
            ent.y = pack_half2(__float2half_rn(c2[(v >> 4) & 3] * s2), __float2half_rn(c2[(v >> 6) & 3] * s2));
            *reinterpret_cast<uint2 *>(g_dyn + v * kLutRow + c * 8) = ent;
        }
        for (int e = tid; e < 64 * 32; e += kMmaThreads) {
            const int idx = e >> 5, c = e & 31;
            *reinterpret_cast<uint32_t *>(g_dyn + idx * kLutRow + 128 + c * 4) =
                pack_half2(__float2half_rn(c3[idx & 7] * s3), __float2half_rn(c3[idx >> 3] * s3));
        }
        for (int e = tid; e < 256; e += kMmaThreads)
            reinterpret_cast<uint32_t *>(g_dyn + kLutBytes)[e] = pack_half2(__float2half_rn(c4[e & 15] * s4), __float2half_rn(c4[e >> 4] * s4));
    }
    // lane constants merged into every table offset: copy (lane % 16) of the 2-bit entries, copy `lane` of the 3-bit ones
    const uint32_t off2 = (lane & 15) * 8, off3 = 128 + lane * 4;
    // head slots of this lane's two columns
    const int h0 = NT == 1 ? 2 * (t & 1) : 2 * t, h1 = h0 + 1;
    const bool owner = NT == 1 ? (t < 2) : true;   // one lane per (g, head pair) publishes

    // The (sample, KV head) units are laid end to end, each n_cta long; CTA c owns [c * BH, (c + 1) * BH) of
    // that line, i.e. the same fraction r0/n_cta .. r1/n_cta of every segment of each unit it overlaps.
    const int n = a.n_cta;
    long long pos = (long long)blockIdx.x * BH;
    const long long end = pos + BH;
    while (pos < end) {
        const int bh = (int)(pos / n), r0 = (int)(pos % n);
        const int r1 = (int)((long long)r0 + (end - pos) < (long long)n ? (long long)r0 + (end - pos) : (long long)n);
        pos += r1 - r0;
        const int slot = blockIdx.x - (int)(((long long)bh * n) / BH);   // index among the CTAs that overlap this unit

        // ---- query B fragments: column g of tile nt; NT = 1: columns 0..3 high limbs, 4..7 low limbs of
        // heads 0..3; NT = 2: tile 0 high limbs, tile 1 low limbs of heads 0..7
        for (int e = tid; e < NH * kD; e += kMmaThreads) (&Osh[0][0])[e] = 0.f;
        if (tid < NH) { lsh[tid] = 0.f; Msh[tid] = kNegBig; }
        if (warp == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int head = NT == 1 ? (g & 3) : g;
                const bool low = NT == 1 ? (g >= 4) : (nt == 1);
                const float *qr = a.qrot + ((size_t)bh * G + (head < G ? head : 0)) * kD + 32 * t;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    __half h[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float v = head < G ? qr[4 * s + e] : 0.f;
                        __half hv = __float2half_rn(v);
                        h[e] = low ? __float2half_rn(v - __half2float(hv)) : hv;
                    }
                    qBs[(nt * 8 + s) * 32 + lane] = make_uint2(pack_half2(h[0], h[1]), pack_half2(h[2], h[3]));
                }
            }
        }
        __syncthreads();

        MmaState<NT> st;
        st.M[0] = st.M[1] = kNegBig;
        st.l[0] = st.l[1] = 0.f;
#pragma unroll
        for (int m = 0; m < 8; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) st.O[m][i] = 0.f;

        for (int ci = 0; ci < chunks.n; ++ci) {
            const odmkv_chunk &ch = chunks.ch[ci];
            for (int c = 1; c <= 3; ++c) {
                const int cnt = ch.seg_count[c * BH + bh];
                if (cnt == 0) continue;
                const int s0 = ch.seg_start[c * BH + bh];
                if (c == 1) process_segment<2, NT>(st, ch, s0, cnt, r0, r1, n, warp, lane, qBs, off2, a.scale_log2, a.lut_scale[0]);
                else if (c == 2) process_segment<3, NT>(st, ch, s0, cnt, r0, r1, n, warp, lane, qBs, off3, a.scale_log2, a.lut_scale[1]);
                else process_segment<4, NT>(st, ch, s0, cnt, r0, r1, n, warp, lane, qBs, 0u, a.scale_log2, a.lut_scale[2]);
            }
        }

        // ---- per-warp totals: denominators summed over the 8 row groups; NT = 1: lanes t and t^2 hold copies
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], o);
            st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], o);
        }
        if (NT == 1) {
            // fold the low-limb columns (lanes t >= 2) into the high-limb lanes
#pragma unroll
            for (int m = 0; m < 8; ++m)
#pragma unroll
                for (int i = 0; i < 4; ++i) st.O[m][i] += __shfl_xor_sync(0xffffffffu, st.O[m][i], 2);
        }
        if (g == 0 && owner) { warpM[warp][h0] = st.M[0]; warpM[warp][h1] = st.M[1]; }
        __syncthreads();
        if (tid < NH) {
            float m = kNegBig;
#pragma unroll
            for (int w = 0; w < kMmaWarps; ++w) m = fmaxf(m, warpM[w][tid]);
            Msh[tid] = m;
        }
        __syncthreads();
        const float c0 = st.M[0] <= kNegBig ? 0.f : fast_exp2(st.M[0] - Msh[h0]);
        const float c1 = st.M[1] <= kNegBig ? 0.f : fast_exp2(st.M[1] - Msh[h1]);
        for (int w = 0; w < kMmaWarps; ++w) {   // fixed order: the sum is reproducible
            if (warp == w && owner) {
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    const float v0 = st.O[m][0], v1 = st.O[m][1], v2 = st.O[m][2], v3 = st.O[m][3];
                    Osh[h0][16 * m + g] += v0 * c0;
                    Osh[h1][16 * m + g] += v1 * c1;
                    Osh[h0][16 * m + g + 8] += v2 * c0;
                    Osh[h1][16 * m + g + 8] += v3 * c1;
                }
                if (g == 0) { lsh[h0] += st.l[0] * c0; lsh[h1] += st.l[1] * c1; }
            }
            __syncthreads();
        }
        // ---- write the partial (natural-log maximum, code-space accumulator; exact-space part is zero)
        const int GP = round_gp(G);
        for (int e = tid; e < GP * 2 * kD; e += kMmaThreads) {
            const int gq = e / (2 * kD), rest = e % (2 * kD);
            const size_t pi = ((size_t)bh * a.nslots + a.slot_base + slot) * GP + gq;
            float v = 0.f;
            if (rest < kD && gq < NH) v = Osh[gq][rest];
            a.part_acc[pi * 2 * kD + rest] = v;
            if (rest == 0) {
                a.part_ml[pi * 2] = (gq < NH && Msh[gq] > kNegBig) ? Msh[gq] * 0.6931471805599453f : -INFINITY;
                a.part_ml[pi * 2 + 1] = gq < NH ? lsh[gq] : 0.f;
            }
        }
        __syncthreads();   // the shared accumulators are reset for the next unit
    }
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

// Shared body of the tensor-core entry points.  With tail_len_dev the kernels read the tail length from device
// memory (plus tail_len_add) and `tail_len` only bounds it for the sizing of the launch.
static int decode_attn_mma_impl(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                                const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                                const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                                int out_dtype, float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                                const float *lut_scales, void *stream, const int32_t *tail_len_dev, int tail_len_add) {
    DecodeChunks dc;
    int rc = decode_check_args(q, q_dtype, chunks, n_chunks, cache_dtype, tail_k, tail_v, tail_len, tail_cap, pi_k, pi_v, codebooks,
                               B, H, G, out, out_dtype, n_splits, workspace, &dc);
    if (rc) return rc;
    // exact / 8-bit / tail tokens: a few CTAs of the CUDA-core kernel per (b, h)
    long long side_tokens = tail_len;
    for (int i = 0; i < n_chunks; ++i) side_tokens += ((long long)chunks[i].cap[4] + chunks[i].cap[5]) / ((long long)B * H) + 1;
    int ns_side = (int)((side_tokens + 127) / 128);   // one 32-token group per warp of the CUDA-core kernel
    if (ns_side < 1) ns_side = 1;
    if (ns_side > 8) ns_side = 8;
    const int nslots = n_splits + ns_side;
    DecodeWs ws;
    if (workspace_bytes < decode_ws_layout(B, H, G, nslots, &ws, (unsigned char *)workspace)) return ODMKV_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int BH = B * H;
    // Without 8-bit codes the exact / tail kernel needs no rotated query: it is forked before the rotation and runs
    // beside it and the start of the tensor-core kernel.
    bool has8 = false;
    for (int i = 0; i < n_chunks; ++i) has8 = has8 || chunks[i].cap[4] > 0;
    SideStream *ss = side_stream();
    // (only while its CTAs are few: with many units they would hold up a noticeable part of the tensor-core grid)
    long long side_tok = tail_len;
    for (int i = 0; i < n_chunks; ++i) side_tok += ((long long)chunks[i].cap[4] + chunks[i].cap[5]) / ((long long)B * H) + 1;
    const long long side_ctas = (long long)B * H * ((side_tok + 127) / 128 < 8 ? (side_tok + 127) / 128 : 8);
    const bool early_side = ss && !has8 && 2 * side_ctas <= num_sms_cached();
    if (early_side) cudaEventRecord(ss->fork, st);
    timing_begin("decode_rotate", st);
    launch_rotate_q(q, q_dtype, pi_k, ws, BH * G, st);
    timing_end(st);
    if (ss && !early_side) cudaEventRecord(ss->fork, st);
    MmaArgs m;
    m.qrot = ws.qrot; m.codebooks = codebooks; m.part_ml = ws.part_ml; m.part_acc = ws.part_acc;
    // grid: one CTA pair per SM, fewer when the cache is short (at least ~32 tiles per CTA) or when the caller's
    // slot count bounds the CTAs that may overlap one unit
    long long total_tiles = 0;
    for (int i = 0; i < n_chunks; ++i) total_tiles += ((long long)chunks[i].cap[1] + chunks[i].cap[2] + chunks[i].cap[3]) / 16;
    long long n_cta = 2ll * num_sms_cached();
    if (n_cta > total_tiles / 32) n_cta = total_tiles / 32;
    if (n_splits >= 2) {
        if (n_cta > (long long)(n_splits - 1) * BH) n_cta = (long long)(n_splits - 1) * BH;
    } else {
        if (n_cta > BH) n_cta = BH;
        while (n_cta > 1 && BH % n_cta != 0) --n_cta;   // one slot: every unit belongs to exactly one CTA
    }
    if (n_cta < 1) n_cta = 1;
    m.B = B; m.H = H; m.G = G; m.n_cta = (int)n_cta; m.slot_base = 0; m.nslots = nslots;
    m.scale_log2 = scale * 1.4426950408889634f;
    for (int i = 0; i < 3; ++i) m.lut_scale[i] = lut_scales ? lut_scales[i] : 1.0f;
    dim3 grid((unsigned)n_cta);
    {
        static bool attr_set[64] = {};   // per device: the opt-in only has to happen once
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            cudaError_t e1 = cudaFuncSetAttribute(decode_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes);
            cudaError_t e2 = cudaFuncSetAttribute(decode_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes);
            if (e1 != cudaSuccess) return (int)e1;
            if (e2 != cudaSuccess) return (int)e2;
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    DecodeArgs a;
    a.qrot = ws.qrot; a.qf = ws.qf; a.tail_k = tail_k; a.tail_v = tail_v; a.codebooks = codebooks;
    a.part_ml = ws.part_ml; a.part_acc = ws.part_acc; a.tail_len = tail_len; a.tail_cap = tail_cap;
    a.tail_len_dev = tail_len_dev; a.tail_len_add = tail_len_add;
    a.B = B; a.H = H; a.G = G; a.nsplit = ns_side; a.slot_base = n_splits; a.nslots = nslots;
    a.class_mask = (1 << 4) | (1 << 5) | (1 << 6); a.scale = scale;
    a.q_raw = early_side ? q : nullptr; a.q_dtype = q_dtype;
    if (early_side) a.class_mask = (1 << 5) | (1 << 6);
    // The exact / tail kernel runs on a second stream, joined before the merge.  The tensor-core kernel fills every SM's
    // registers, so the small kernel either starts before it (forked before the rotation, when it does not need the
    // rotated queries) or slips into its tail as CTAs retire.
    auto launch_side = [&]() {
        cudaStreamWaitEvent(ss->stream, ss->fork, 0);
        timing_begin("decode_side", ss->stream);
        launch_decode_cuda_core(dc, a, cache_dtype, ss->stream);
        timing_end(ss->stream);
        cudaEventRecord(ss->join, ss->stream);
    };
    if (early_side) launch_side();
    timing_begin("decode_main", st);
    if (G <= 4) decode_mma_kernel<1><<<grid, kMmaThreads, kStageBytes, st>>>(dc, m);
    else decode_mma_kernel<2><<<grid, kMmaThreads, kStageBytes, st>>>(dc, m);
    timing_end(st);
    if (ss && !early_side) launch_side();
    if (ss) {
        cudaStreamWaitEvent(st, ss->join, 0);
    } else {
        timing_begin("decode_side", st);
        launch_decode_cuda_core(dc, a, cache_dtype, st);
        timing_end(st);
    }
    timing_begin("decode_merge", st);
    launch_decode_merge(ws, pi_v, BH, G, nslots, out, out_dtype, lse, st, n_splits, (int)n_cta);
    timing_end(st);
    return launch_status();
}

extern "C" {

// Same arguments as odmkv_decode_attn plus `lut_scales` (host float[3] or NULL for 1.0): per level a
// factor s such that fp16(c * s) represents the centroids of the 2-, 3- and 4-bit codebooks with less
// rounding error than fp16(c); the kernel divides it out again in fp32.
int odmkv_decode_attn_mma(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                          const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                          const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                          int out_dtype, float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                          const float *lut_scales, void *stream) {
    return decode_attn_mma_impl(q, q_dtype, chunks, n_chunks, cache_dtype, tail_k, tail_v, tail_len, tail_cap, pi_k, pi_v, codebooks,
                                B, H, G, scale, out, out_dtype, lse, n_splits, workspace, workspace_bytes, lut_scales, stream,
                                nullptr, 0);
}

// The same call with the tail length in device memory: the launch attends min(*tail_len_dev + tail_len_add,
// tail_cap) tail tokens, so one captured launch stays valid while a counter on the device advances.
int odmkv_decode_attn_mma_devtail(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                                  const void *tail_k, const void *tail_v, const int32_t *tail_len_dev, int tail_len_add,
                                  int tail_len_bound, int tail_cap, const float *pi_k, const float *pi_v,
                                  const float *codebooks, int B, int H, int G, float scale, void *out, int out_dtype,
                                  float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                                  const float *lut_scales, void *stream) {
    if (!tail_len_dev || !tail_k || !tail_v || tail_len_add < 0 || tail_len_bound < 1 || tail_len_bound > tail_cap) return ODMKV_ERR_ARG;
    return decode_attn_mma_impl(q, q_dtype, chunks, n_chunks, cache_dtype, tail_k, tail_v, tail_len_bound, tail_cap, pi_k, pi_v,
                                codebooks, B, H, G, scale, out, out_dtype, lse, n_splits, workspace, workspace_bytes, lut_scales,
                                stream, tail_len_dev, tail_len_add);
}

}  // extern "C"
