// Quantise-and-pack, dequantise and bank export kernels (sm_100a).
//
// Replaces the reference's routing + TurboQuantMSE path (kvquant/tq_adaptive_backend.py:350-374,
// 149-174, 205-242; kvquant/tq_backend.py:103-145, 185-203).  The 128x128 rotation of a 32-token item runs on the
// tensor cores (mma.sync, operands as fp16 high/low limb pairs, three products, fp32 accumulate); every coordinate
// whose distance to a decision boundary is inside the proven error margin is recomputed with one ascending fp32
// fused-multiply-add chain over the contraction index -- the chain the CPU oracle uses -- so codes are reproducible
// bit for bit.
#include "common.cuh"

namespace odmkv {

constexpr int kLd = 132;  // padded fp32 row stride in shared memory (conflict-free 128-bit reads)
constexpr int kLdC = 144; // byte row stride of the staged codes

// ----------------------------------------------------------------------------------------------
// Plan: per-tile class counts, exclusive scans, segment table
// ----------------------------------------------------------------------------------------------
__global__ void count_tiles_kernel(const int32_t *__restrict__ bits, int T, int ntiles,
                                   int32_t *__restrict__ tile_counts, int32_t *__restrict__ totals) {
    const int tile = blockIdx.x, bh = blockIdx.y;
    const int t = tile * kTile + threadIdx.x;
    int c = -2;
    if (t < T) c = class_of_bits(bits[(size_t)bh * T + t]);
    __shared__ int cnt[4][kNumClasses];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int cc = 0; cc < kNumClasses; ++cc) {
        unsigned m = __ballot_sync(0xffffffffu, c == cc);
        if (lane == 0) cnt[warp][cc] = __popc(m);
    }
    unsigned bad = __ballot_sync(0xffffffffu, c == -1);
    if (lane == 0 && bad) atomicAdd(&totals[6], __popc(bad));
    __syncthreads();
    if (threadIdx.x < kNumClasses) {
        int s = cnt[0][threadIdx.x] + cnt[1][threadIdx.x] + cnt[2][threadIdx.x] + cnt[3][threadIdx.x];
        tile_counts[((size_t)bh * ntiles + tile) * kNumClasses + threadIdx.x] = s;
    }
}

__device__ inline int warp_incl_scan(int v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

// one block per (b, h); warp c scans the tiles of class c
__global__ void scan_tiles_kernel(const int32_t *__restrict__ tile_counts, int ntiles, int BH,
                                  int32_t *__restrict__ tile_base, int32_t *__restrict__ seg_count) {
    const int bh = blockIdx.x, c = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int carry = 0;
    for (int base = 0; base < ntiles; base += 32) {
        int tile = base + lane;
        int v = tile < ntiles ? tile_counts[((size_t)bh * ntiles + tile) * kNumClasses + c] : 0;
        int incl = warp_incl_scan(v, lane);
        if (tile < ntiles) tile_base[((size_t)bh * ntiles + tile) * kNumClasses + c] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) seg_count[c * BH + bh] = carry;
}

// one block; warp c lays out the (b, h) segments of class c on 16-slot boundaries
__global__ void scan_segs_kernel(const int32_t *__restrict__ seg_count, int BH, int32_t *__restrict__ seg_start,
                                 int32_t *__restrict__ totals) {
    const int c = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int carry = 0;
    for (int base = 0; base < BH; base += 32) {
        int bh = base + lane;
        int v = bh < BH ? ((seg_count[c * BH + bh] + kSegAlign - 1) / kSegAlign) * kSegAlign : 0;
        int incl = warp_incl_scan(v, lane);
        if (bh < BH) seg_start[c * BH + bh] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) totals[c] = carry;
}

// ----------------------------------------------------------------------------------------------
// Quantise kernel
// ----------------------------------------------------------------------------------------------
struct QuantArgs {
    const void *K;
    const void *V;
    const int32_t *bits;
    const float *pi_k;
    const float *pi_v;
    const float *codebooks;
    const int32_t *tile_base;
    uint8_t *k_scratch[3];   // linear-layout codes of the 2/3/4-bit banks before re-tiling
    uint8_t *v_scratch[3];
    odmkv_chunk ch;
    int ntiles;
};

// 128x128x128 product: acc[a][b] = sum_i X[ty+16a][i] * P[tx+16b][i], ascending i, one FMA chain each
__device__ inline void tile_product(const float *__restrict__ Xs, const float *__restrict__ Ps, int ty, int tx,
                                    float (&acc)[8][8]) {
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0.0f;
    const float *xrow = Xs + ty * kLd;
    const float *prow = Ps + tx * kLd;
#pragma unroll 1
    for (int i4 = 0; i4 < kD / 4; ++i4) {
        float4 xa[8], pb[8];
#pragma unroll
        for (int a = 0; a < 8; ++a) xa[a] = *reinterpret_cast<const float4 *>(xrow + a * 16 * kLd + 4 * i4);
#pragma unroll
        for (int b = 0; b < 8; ++b) pb[b] = *reinterpret_cast<const float4 *>(prow + b * 16 * kLd + 4 * i4);
#pragma unroll
        for (int a = 0; a < 8; ++a)
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                float v = acc[a][b];
                v = fmaf(xa[a].x, pb[b].x, v);
                v = fmaf(xa[a].y, pb[b].y, v);
                v = fmaf(xa[a].z, pb[b].z, v);
                v = fmaf(xa[a].w, pb[b].w, v);
                acc[a][b] = v;
            }
    }
}

// Pack four staged codes per lane.  `j` is the lane's position inside the destination bit stream (each
// lane contributes 4*b bits at bit offset 4*b*j); called by a full warp.
__device__ inline void pack_lane_codes(const uint8_t *__restrict__ row, int li, uint8_t *__restrict__ dst, int lane, int j) {
    const uint32_t c0 = row[4 * lane], c1 = row[4 * lane + 1], c2 = row[4 * lane + 2], c3 = row[4 * lane + 3];
    if (li == 0) {
        dst[j] = (uint8_t)((c0 & 3) | ((c1 & 3) << 2) | ((c2 & 3) << 4) | ((c3 & 3) << 6));
    } else if (li == 1) {
        const uint32_t v = (c0 & 7) | ((c1 & 7) << 3) | ((c2 & 7) << 6) | ((c3 & 7) << 9);
        const uint32_t nxt = __shfl_down_sync(0xffffffffu, v, 1);
        if ((j & 1) == 0) {
            const uint32_t w = v | (nxt << 12);
            uint8_t *q = dst + 3 * (j >> 1);
            q[0] = (uint8_t)w; q[1] = (uint8_t)(w >> 8); q[2] = (uint8_t)(w >> 16);
        }
    } else if (li == 2) {
        *reinterpret_cast<uint16_t *>(dst + 2 * j) = (uint16_t)((c0 & 15) | ((c1 & 15) << 4) | ((c2 & 15) << 8) | ((c3 & 15) << 12));
    } else {
        *reinterpret_cast<uint32_t *>(dst + 4 * j) = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
    }
}

// codes of one slot in the linear layout (scratch for 2/3/4 bits, final for 8 bits)
__device__ inline void store_linear_codes(const uint8_t *__restrict__ row, int li, uint8_t *__restrict__ rows, long long slot, int lane) {
    pack_lane_codes(row, li, rows + (size_t)slot * 16 * qbits(li), lane, lane);
}

constexpr int kQRows = 32;      // tokens per work item of quantize_kernel: a quarter of a plan tile
constexpr int kGroups = 4;      // independent groups per CTA
constexpr int kGroupThreads = 128;
constexpr int kLdH = 136;    // padded fp16 row stride (272 bytes: conflict-free ldmatrix rows)

// Decision margin of the tensor-core pass.  The rotation is first evaluated on the tensor cores with every
// operand split into an fp16 high and low limb (x = xh + xl, p = ph + pl) and the three products xh ph + xh pl +
// xl ph accumulated in fp32.  With |x_unit| <= 1 and |row of Pi| = 1 (so sum|x_i p_i| <= 1 by Cauchy-Schwarz) the
// result differs from the fp32 FMA chain by at most
//     2^-22 sum|x p|                       (the dropped xl pl term)
//   + 2 * 2^-21.5 sum|x p| + 7e-7          (what the low limbs miss: 11 bits each, 2^-25 absolute when subnormal)
//   + 24 * 2^-22 + 8 * 16 * 2^-23          (fp32 accumulation of 24 HMMA steps, generous)
//   + 128 * 2^-24                          (the chain's own error)
//   < 3e-5.
// The decision itself runs in fp16 against fp16 midpoints of adjacent centroids: both roundings cost at most
// 2^-14 each for |y| < 0.25 (every midpoint of the 2/3/4-bit codebooks is below 0.22).  A coordinate closer than
// kTcMarginBits (1.6e-4 >= 3e-5 + 2 * 6.1e-5) to a midpoint is recomputed with the exact chain and the exact
// rule, so every emitted code equals the code of the chain.
constexpr uint32_t kTcMarginBits = 0x093f093fu;   // half2 {1.601e-4, 1.601e-4}

// per-level constants of the fp16 decision: positive midpoints (padded with +inf) and the code offset
struct LevelConst {
    uint32_t mid[7];   // half2 broadcast
    uint32_t base;     // half2 broadcast of 512 + K/2 - 0.5
};

__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// Two coordinates at once.  Returns the fp16 pair 512 + code (so code = (bits >> 1) & 15 per half); `ok`
// holds 1.0 per half whose distance to every midpoint (and to zero) is at least the margin.
template <int NM>
__device__ __forceinline__ uint32_t decide_pair(uint32_t y2, const uint32_t (&mid)[7], uint32_t base, uint32_t &ok) {
    const __half2 ay = __habs2(u2h(y2));
    __half2 cnt = __hgt2(ay, u2h(mid[0]));
    __half2 d = __hmin2(ay, __habs2(__hsub2(ay, u2h(mid[0]))));
#pragma unroll
    for (int j = 1; j < NM; ++j) {
        cnt = __hadd2(cnt, __hgt2(ay, u2h(mid[j])));
        d = __hmin2(d, __habs2(__hsub2(ay, u2h(mid[j]))));
    }
    const uint32_t sgn = (y2 & 0x80008000u) | 0x3c003c00u;   // +-1.0
    const __half2 cf = __hfma2(u2h(sgn), __hadd2(cnt, u2h(0x38003800u)), u2h(base));
    ok = h2u(__hge2(d, u2h(kTcMarginBits)));                  // NaN compares false
    return h2u(cf);
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void hmma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// the 16-byte pieces of a quarter tile that one thread moves (32 rows of 128 elements, 128 threads)
template <int DT>
struct RawPieces {
    static constexpr int kN = (DT == kF32) ? 8 : 4;
    uint4 v[kN];
};

template <int DT>
__device__ __forceinline__ void load_pieces(const void *__restrict__ src, size_t row0, int rows_left, int tid, RawPieces<DT> &r) {
    constexpr int kPerRow = (DT == kF32) ? 32 : 16;   // pieces per row
    const uint4 *base = reinterpret_cast<const uint4 *>(reinterpret_cast<const unsigned char *>(src) +
                                                        row0 * sizeof(typename Elem<DT>::T));
#pragma unroll
    for (int u = 0; u < RawPieces<DT>::kN; ++u) {
        const int g = tid + kGroupThreads * u, row = g / kPerRow;
        r.v[u] = row < rows_left ? __ldg(base + g) : make_uint4(0u, 0u, 0u, 0u);
    }
}

template <int DT>
__device__ __forceinline__ void store_pieces_f32(const RawPieces<DT> &r, int tid, float *__restrict__ Xs) {
    constexpr int kPerRow = (DT == kF32) ? 32 : 16;
#pragma unroll
    for (int u = 0; u < RawPieces<DT>::kN; ++u) {
        const int g = tid + kGroupThreads * u, row = g / kPerRow, pc = g % kPerRow;
        const uint32_t w[4] = {r.v[u].x, r.v[u].y, r.v[u].z, r.v[u].w};
        if constexpr (DT == kF32) {
            *reinterpret_cast<float4 *>(Xs + row * kLd + 4 * pc) =
                make_float4(__uint_as_float(w[0]), __uint_as_float(w[1]), __uint_as_float(w[2]), __uint_as_float(w[3]));
        } else {
            float f[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 t2;
                if constexpr (DT == kF16) t2 = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
                else t2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[k]));
                f[2 * k] = t2.x; f[2 * k + 1] = t2.y;
            }
            *reinterpret_cast<float4 *>(Xs + row * kLd + 8 * pc) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4 *>(Xs + row * kLd + 8 * pc + 4) = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
}

// overwrite the b-bit code of coordinate `col` in a packed row held in shared memory
__device__ __forceinline__ void patch_code(uint32_t *__restrict__ row_words, int b, int col, uint32_t code) {
    const int bit = b * col, wi = bit >> 5, sh = bit & 31;
    const uint32_t mask = (1u << b) - 1u;
    atomicAnd(row_words + wi, ~(mask << sh));
    atomicOr(row_words + wi, code << sh);
    if (sh + b > 32) {
        atomicAnd(row_words + wi + 1, ~(mask >> (32 - sh)));
        atomicOr(row_words + wi + 1, code >> (32 - sh));
    }
}

// One CTA serves one side (even blocks: keys, odd blocks: values) with four independent groups of 128
// threads; each group walks over quarter tiles of 32 tokens with its own buffers and its own named barrier,
// so the latency-bound steps of one group run under the arithmetic of the other.  The fp16 high and low limbs
// of the side's rotation (for the tensor cores) are shared by both groups; the exact chains read its fp32 rows
// from global memory (a few dozen rows per item).
// Per item: rows -> fp32 shared tile; norm (one ascending FMA chain per row, IEEE square root); IEEE
// division; the 64x128x128 rotation on the tensor cores (fp16 limb pairs, three products); an fp16 decision per
// coordinate, packed straight into the row's bit stream in shared memory (a thread owns eight consecutive
// coordinates of a row); every coordinate closer to a decision boundary than the tensor-core error bound
// is queued and recomputed with the exact fp32 chain (ascending contraction index, one FMA per term) and
// the exact nearest-centroid rule, then patched into the packed row -- so the codes are those of the
// chain, bit for bit; copy-out.  The next item's rows, bit widths and slot bases are fetched into
// registers under the decision step of the current one.
constexpr int kQueueCap = 512;    // queued coordinates per item (about 30 are expected); beyond that the whole item is redone exactly
constexpr size_t kQuantGroupSmem = (size_t)(kQRows * kLd + kQRows) * sizeof(float) + kQRows * sizeof(double) + 2 * (size_t)kQRows * kLdH * 2 +
                                   (2 * kTile + 4 * kNumClasses + 16) * sizeof(int) + (size_t)kQueueCap * 2;
constexpr size_t kQuantKernelSmem = (size_t)(4 * 256) * sizeof(float) + 2 * (size_t)kD * kLdH * 2 + 3 * sizeof(LevelConst) +
                                    kGroups * kQuantGroupSmem;

__device__ __forceinline__ void group_sync(int gid) {
    asm volatile("bar.sync %0, 128;\n" ::"r"(gid + 1) : "memory");
}

template <int DT>
__global__ void __launch_bounds__(512, 1) quantize_kernel(const QuantArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *cb = reinterpret_cast<float *>(smem_raw);                 // [4][256]
    __half *Ph = reinterpret_cast<__half *>(cb + 4 * 256);           // [128][kLdH] fp16 high limbs of the rotation, rows permuted
    __half *Pl = Ph + kD * kLdH;                                     // [128][kLdH] fp16 low limbs
    LevelConst *lc = reinterpret_cast<LevelConst *>(Pl + kD * kLdH); // [3] 2, 3, 4 bits
    const int gid = threadIdx.x >> 7, tid = threadIdx.x & 127;       // group, thread within the group
    unsigned char *gbase = reinterpret_cast<unsigned char *>(lc + 3) + (size_t)gid * kQuantGroupSmem;
    float *Xs = reinterpret_cast<float *>(gbase);                    // [32][kLd] fp32 rows, normalised in place
    float *nrm = Xs + kQRows * kLd;                                  // [32]
    double *rinv = reinterpret_cast<double *>(nrm + kQRows);         // [32] 1 / (norm + 1e-10) in fp64
    __half *Xh = reinterpret_cast<__half *>(rinv + kQRows);          // [32][kLdH] fp16 high limbs of the normalised rows
    __half *Xl = Xh + kQRows * kLdH;                                 // [32][kLdH] fp16 low limbs
    int *cls = reinterpret_cast<int *>(Xl + kQRows * kLdH);          // [128]
    int *slot = cls + kTile;                                         // [128]
    int *wcnt = slot + kTile;                                        // [4][6]
    int *tbase = wcnt + 4 * kNumClasses;                             // [8] slot base of this plan tile per class
    int *flags = tbase + 8;                                          // [0] any quantised row, [1] queue length
    uint16_t *queue = reinterpret_cast<uint16_t *>(flags + 8);       // [kQueueCap] coordinates to recompute
    unsigned char *PK = reinterpret_cast<unsigned char *>(Xh);       // [32][kLdC] packed rows (after the product)

    const int lane = tid & 31, warp = tid >> 5;
    const int B = a.ch.B, H = a.ch.H, T = a.ch.T, BH = B * H;
    const int side = blockIdx.x & 1;
    const void *src = side ? a.V : a.K;
    const float *pi = side ? a.pi_v : a.pi_k;
    // shared row q of the fp16 rotation holds row j(q) of Pi, chosen so that the eight tensor-core columns
    // a thread owns per 32-column window are eight consecutive coordinates:
    //   q = 32 wn + 8 nb + n  ->  j = 32 wn + 8 (n >> 1) + 2 nb + (n & 1)
    for (int g = threadIdx.x; g < kD * kD / 4; g += 512) {
        const int q = g >> 5, i4 = g & 31;
        const int j = (q & ~31) + 8 * ((q & 7) >> 1) + 2 * ((q >> 3) & 3) + (q & 1);
        const float4 f = *reinterpret_cast<const float4 *>(pi + j * kD + 4 * i4);
        const __half2 h01 = __floats2half2_rn(f.x, f.y), h23 = __floats2half2_rn(f.z, f.w);
        __half2 *dst = reinterpret_cast<__half2 *>(Ph + q * kLdH + 4 * i4);
        dst[0] = h01;
        dst[1] = h23;
        const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
        __half2 *dlo = reinterpret_cast<__half2 *>(Pl + q * kLdH + 4 * i4);
        dlo[0] = __floats2half2_rn(f.x - b01.x, f.y - b01.y);
        dlo[1] = __floats2half2_rn(f.z - b23.x, f.w - b23.y);
    }
    for (int g = threadIdx.x; g < 4 * 256; g += 512) cb[g] = a.codebooks[g];
    if (threadIdx.x < 3 * 8) {
        const int li = threadIdx.x >> 3, j = threadIdx.x & 7, half_k = 1 << (li + 1);   // K/2 for 2, 3, 4 bits
        const float *cbl = a.codebooks + li * 256;
        if (j < 7) {
            __half m = __ushort_as_half((unsigned short)0x7c00);        // +inf: never exceeded, never near
            if (j + 1 < half_k) m = __float2half_rn(0.5f * (cbl[half_k + j] + cbl[half_k + j + 1]));
            lc[li].mid[j] = h2u(__half2half2(m));
        } else {
            lc[li].base = h2u(__half2half2(__float2half_rn(512.0f + (float)half_k - 0.5f)));
        }
    }

    const long long n_work = (long long)BH * a.ntiles * 4;
    const long long w_step = (long long)(gridDim.x >> 1) * kGroups;   // four groups per CTA, half of the CTAs per side
    const long long w_first = (long long)(blockIdx.x >> 1) * kGroups + gid;
    // fetched ahead: rows, this thread's bit width (threads < 128) and slot base (threads < 6)
    RawPieces<DT> raw;
    int pf_bits = 0, pf_base = 0;
    auto prefetch = [&](long long w) {
        if (w >= n_work) return;
        const int bh = (int)(w / (4 * a.ntiles)), rem = (int)(w % (4 * a.ntiles));
        const int tile = rem >> 2, half = rem & 3;
        const int t0 = tile * kTile, h0 = half * kQRows;
        if (t0 + h0 >= T) return;
        load_pieces<DT>(src, ((size_t)bh * T + t0 + h0) * kD, T - t0 - h0, tid, raw);
        if (tid < kTile) pf_bits = (t0 + tid < T) ? a.bits[(size_t)bh * T + t0 + tid] : -1;
        if (tid < kNumClasses)
            pf_base = a.ch.seg_start[tid * BH + bh] + a.tile_base[((size_t)bh * a.ntiles + tile) * kNumClasses + tid];
    };
    prefetch(w_first);
    __syncthreads();

    // tensor-core tiling: warp wn owns the item's 32 rows and columns [32 wn, +32)
    const int wm = 0, wn = warp, g8 = lane >> 2, t4 = lane & 3;

    for (long long w = w_first; w < n_work; w += w_step) {
        const int bh = (int)(w / (4 * a.ntiles)), rem = (int)(w % (4 * a.ntiles));
        const int tile = rem >> 2, half = rem & 3;
        const int t0 = tile * kTile, h0 = half * kQRows;
        if (t0 + h0 >= T) { prefetch(w + w_step); continue; }
        if (tid == 0) { flags[0] = 0; flags[1] = 0; }
        // ---- classes and slots of the whole plan tile (the slot of a token counts the tokens before it)
        int c = -1, rank = 0;
        if (tid < kTile) {
            if (t0 + tid < T) c = class_of_bits(pf_bits);
#pragma unroll
            for (int cc = 0; cc < kNumClasses; ++cc) {
                unsigned m = __ballot_sync(0xffffffffu, c == cc);
                if (c == cc) rank = __popc(m & ((1u << lane) - 1u));
                if (lane == 0) wcnt[warp * kNumClasses + cc] = __popc(m);
            }
            if (tid < kNumClasses) tbase[tid] = pf_base;
        }
        store_pieces_f32<DT>(raw, tid, Xs);
        group_sync(gid);
        if (tid < kTile) {
            int s = -1;
            if (c >= 0) {
                s = tbase[c] + rank;
                for (int ww = 0; ww < warp; ++ww) s += wcnt[ww * kNumClasses + c];
                if (c >= 1 && c <= 4 && (tid >> 5) == half) flags[0] = 1;
            }
            cls[tid] = c;
            slot[tid] = s;
        }
        // ---- fp32 norm: one ascending FMA chain of squares, IEEE square root
        if (tid >= kGroupThreads - kQRows) {
            const int r = tid - (kGroupThreads - kQRows);
            float acc = 0.0f;
            const float *xr = Xs + r * kLd;
#pragma unroll 8
            for (int i4 = 0; i4 < kD / 4; ++i4) {
                float4 v = *reinterpret_cast<const float4 *>(xr + 4 * i4);
                acc = fmaf(v.x, v.x, acc);
                acc = fmaf(v.y, v.y, acc);
                acc = fmaf(v.z, v.z, acc);
                acc = fmaf(v.w, v.w, acc);
            }
            const float nr = __fsqrt_rn(acc);
            nrm[r] = nr;
            rinv[r] = 1.0 / (double)__fadd_rn(nr, 1e-10f);
        }
        group_sync(gid);
        const bool any_q = flags[0] != 0;
        const size_t row0 = ((size_t)bh * T + t0 + h0) * kD;
        if (any_q) {
            // ---- x / (norm + 1e-10) as the IEEE fp32 quotient, computed as fp32(fp64(x) * fp64(1 / den)): the fp64
            //      product is within 2^-52 of the quotient, while a quotient of two fp32 numbers is never closer
            //      than 2^-49 (relative) to a rounding boundary of fp32 and never on one, so the final rounding
            //      lands where the division's would.  fp32 result in place, fp16 copy for the tensor cores.
            {
                // all loads first, then the arithmetic, then the stores: the eight pieces of a thread are independent
                constexpr int kPieces = kQRows * kD / 4 / kGroupThreads;
                float4 v[kPieces];
                double ri[kPieces];
#pragma unroll
                for (int u = 0; u < kPieces; ++u) {
                    const int g = tid + kGroupThreads * u, r = g >> 5, i4 = g & 31;
                    v[u] = *reinterpret_cast<const float4 *>(Xs + r * kLd + 4 * i4);
                    ri[u] = rinv[r];
                }
#pragma unroll
                for (int u = 0; u < kPieces; ++u) {
                    v[u].x = __double2float_rn(__dmul_rn((double)v[u].x, ri[u]));
                    v[u].y = __double2float_rn(__dmul_rn((double)v[u].y, ri[u]));
                    v[u].z = __double2float_rn(__dmul_rn((double)v[u].z, ri[u]));
                    v[u].w = __double2float_rn(__dmul_rn((double)v[u].w, ri[u]));
                }
#pragma unroll
                for (int u = 0; u < kPieces; ++u) {
                    const int g = tid + kGroupThreads * u, r = g >> 5, i4 = g & 31;
                    *reinterpret_cast<float4 *>(Xs + r * kLd + 4 * i4) = v[u];
                    const __half2 h01 = __floats2half2_rn(v[u].x, v[u].y), h23 = __floats2half2_rn(v[u].z, v[u].w);
                    const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
                    uint2 hw, lw;
                    hw.x = h2u(h01); hw.y = h2u(h23);
                    lw.x = h2u(__floats2half2_rn(v[u].x - b01.x, v[u].y - b01.y));
                    lw.y = h2u(__floats2half2_rn(v[u].z - b23.x, v[u].w - b23.y));
                    *reinterpret_cast<uint2 *>(Xh + r * kLdH + 4 * i4) = hw;
                    *reinterpret_cast<uint2 *>(Xl + r * kLdH + 4 * i4) = lw;
                }
            }
            group_sync(gid);
            // ---- approximate rotation on the tensor cores: acc[mb][nb] = 16x8 block of X Pi^T
            float acc[2][4][4];
#pragma unroll
            for (int mb = 0; mb < 2; ++mb)
#pragma unroll
                for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[mb][nb][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < kD / 16; ++ks) {
                uint32_t ah[2][4], al[2][4], bh[2][4], bl[2][4];
#pragma unroll
                for (int mb = 0; mb < 2; ++mb) {
                    const int off = (32 * wm + 16 * mb + (lane & 15)) * kLdH + 16 * ks + 8 * (lane >> 4);
                    ldmatrix_x4(ah[mb], Xh + off);
                    ldmatrix_x4(al[mb], Xl + off);
                }
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    const int off = (32 * wn + 16 * np + 8 * (lane >> 4) + (lane & 7)) * kLdH + 16 * ks + 8 * ((lane >> 3) & 1);
                    ldmatrix_x4(bh[np], Ph + off);
                    ldmatrix_x4(bl[np], Pl + off);
                }
#pragma unroll
                for (int mb = 0; mb < 2; ++mb)
#pragma unroll
                    for (int nb = 0; nb < 4; ++nb) {
                        const int np = nb >> 1, o = 2 * (nb & 1);
                        hmma_16816(acc[mb][nb], al[mb], bh[np][o], bh[np][o + 1]);
                        hmma_16816(acc[mb][nb], ah[mb], bl[np][o], bl[np][o + 1]);
                        hmma_16816(acc[mb][nb], ah[mb], bh[np][o], bh[np][o + 1]);
                    }
            }
            group_sync(gid);   // every warp is done with Xh: the packed rows reuse its space
            prefetch(w + w_step);
            // ---- fp16 decision and packing; this thread's coordinates of a row are 32 wn + 8 t4 + [0, 8),
            //      element (nb, e) of the accumulator being coordinate 2 nb + e of those.  The four rows of a
            //      thread go through one branch-free path for 2 and 3 bits (a 2-bit row pads its midpoints with
            //      +inf); 4- and 8-bit rows are redone afterwards.
            {
                const int col0 = 32 * wn + 8 * t4;
                int ccs[4];
                uint32_t words[4], bads[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) ccs[k] = cls[h0 + 32 * wm + 16 * (k >> 1) + g8 + 8 * (k & 1)];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int mb = k >> 1, hi = k & 1;
                    const LevelConst &L = lc[ccs[k] == 2 ? 1 : 0];
                    uint32_t mid[7];
#pragma unroll
                    for (int j = 0; j < 3; ++j) mid[j] = L.mid[j];
                    const uint32_t base = L.base;
                    const int b = ccs[k] == 2 ? 3 : 2;
                    uint32_t word = 0, bad = 0;
#pragma unroll
                    for (int nb = 0; nb < 4; ++nb) {
                        const uint32_t y2 = h2u(__floats2half2_rn(acc[mb][nb][2 * hi], acc[mb][nb][2 * hi + 1]));
                        uint32_t ok;
                        const uint32_t cf = decide_pair<3>(y2, mid, base, ok);
                        const uint32_t field = ((cf >> 1) & 15u) | (((cf >> 17) & 15u) << b);
                        word |= field << (2 * b * nb);
                        if ((ok & 0xffffu) != 0x3c00u) bad |= 1u << (2 * nb);
                        if ((ok >> 16) != 0x3c00u) bad |= 2u << (2 * nb);
                    }
                    words[k] = word;
                    bads[k] = bad;
                }
                bool rare = false;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int r = 32 * wm + 16 * (k >> 1) + g8 + 8 * (k & 1);
                    unsigned char *dst = PK + r * kLdC + (ccs[k] + 1) * (4 * wn + t4);
                    if (ccs[k] == 1) *reinterpret_cast<uint16_t *>(dst) = (uint16_t)words[k];
                    else if (ccs[k] == 2) { dst[0] = (unsigned char)words[k]; dst[1] = (unsigned char)(words[k] >> 8); dst[2] = (unsigned char)(words[k] >> 16); }
                    else if (ccs[k] == 3 || ccs[k] == 4) rare = true;
                    if (ccs[k] == 1 || ccs[k] == 2) {
                        uint32_t bad = bads[k];
                        while (bad) {
                            const int c8 = __ffs(bad) - 1;
                            bad &= bad - 1;
                            const int qi = atomicAdd(&flags[1], 1);
                            if (qi < kQueueCap) queue[qi] = (uint16_t)((r << 7) | (col0 + c8));
                        }
                    }
                }
                if (rare) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int mb = k >> 1, hi = k & 1;
                        const int r = 32 * wm + 16 * mb + g8 + 8 * hi;
                        if (ccs[k] == 4) {   // 8 bits: the centroid spacing is within the margin, every coordinate is exact work
                            for (int c8 = 0; c8 < 8; ++c8) {
                                const int qi = atomicAdd(&flags[1], 1);
                                if (qi < kQueueCap) queue[qi] = (uint16_t)((r << 7) | (col0 + c8));
                            }
                        } else if (ccs[k] == 3) {
                            const LevelConst &L = lc[2];
                            uint32_t mid[7];
#pragma unroll
                            for (int j = 0; j < 7; ++j) mid[j] = L.mid[j];
                            uint32_t word = 0, bad = 0;
#pragma unroll
                            for (int nb = 0; nb < 4; ++nb) {
                                const uint32_t y2 = h2u(__floats2half2_rn(acc[mb][nb][2 * hi], acc[mb][nb][2 * hi + 1]));
                                uint32_t ok;
                                const uint32_t cf = decide_pair<7>(y2, mid, L.base, ok);
                                word |= (((cf >> 1) & 15u) | (((cf >> 17) & 15u) << 4)) << (8 * nb);
                                if ((ok & 0xffffu) != 0x3c00u) bad |= 1u << (2 * nb);
                                if ((ok >> 16) != 0x3c00u) bad |= 2u << (2 * nb);
                            }
                            *reinterpret_cast<uint32_t *>(PK + r * kLdC + 4 * (4 * wn + t4)) = word;
                            while (bad) {
                                const int c8 = __ffs(bad) - 1;
                                bad &= bad - 1;
                                const int qi = atomicAdd(&flags[1], 1);
                                if (qi < kQueueCap) queue[qi] = (uint16_t)((r << 7) | (col0 + c8));
                            }
                        }
                    }
                }
            }
            group_sync(gid);
            // ---- exact recomputation of the queued coordinates: ascending fp32 FMA chain, exact rule
            const int qn = flags[1];
            const bool redo_all = qn > kQueueCap;   // queue overflow: every coordinate of the item is exact work
            const int n_fix = redo_all ? kQRows * kD : qn;
            for (int e = tid; e < n_fix; e += kGroupThreads) {
                const int r = redo_all ? (e >> 7) : (queue[e] >> 7), col = redo_all ? (e & 127) : (queue[e] & 127);
                const int li = cls[h0 + r] - 1;
                if (li < 0 || li > 3) continue;
                const float4 *xr = reinterpret_cast<const float4 *>(Xs + r * kLd);
                const float4 *pr = reinterpret_cast<const float4 *>(pi + col * kD);   // few entries: read through L2
                float y = 0.0f;
#pragma unroll 8
                for (int i = 0; i < kD / 4; ++i) {
                    const float4 xv = xr[i], pv = __ldg(pr + i);
                    y = fmaf(xv.x, pv.x, y);
                    y = fmaf(xv.y, pv.y, y);
                    y = fmaf(xv.z, pv.z, y);
                    y = fmaf(xv.w, pv.w, y);
                }
                const int code = nearest_centroid(y, cb + li * 256, 1 << bits_of_qlevel(li));
                patch_code(reinterpret_cast<uint32_t *>(PK + r * kLdC), qbits(li), col, (uint32_t)code);
            }
            group_sync(gid);
        } else {
            prefetch(w + w_step);
        }
        // ---- copy-out: four threads per row, each moves a quarter of the row
        {
            const int r = tid >> 2, qt = tid & 3;
            const int cc = cls[h0 + r];
            const int s = slot[h0 + r];
            const int t_abs = a.ch.t_offset + t0 + h0 + r;
            if (cc >= 1 && cc <= 4) {
                const int li = cc - 1, nw = qbits(li);   // words per quarter row
                uint8_t *rows = side ? (li == 3 ? a.ch.v_codes[3] : a.v_scratch[li]) : (li == 3 ? a.ch.k_codes[3] : a.k_scratch[li]);
                uint32_t *dst = reinterpret_cast<uint32_t *>(rows + (size_t)s * 16 * nw) + qt * nw;
                const uint32_t *srcw = reinterpret_cast<const uint32_t *>(PK + r * kLdC) + qt * nw;
                for (int k = 0; k < nw; ++k) dst[k] = srcw[k];
                if (qt == 0) {
                    (side ? a.ch.v_norm[li] : a.ch.k_norm[li])[s] = nrm[r];
                    if (side == 0) a.ch.pos[li][s] = t_abs;
                }
            } else if (cc == 5) {
                constexpr int kVec = (int)(kD * sizeof(typename Elem<DT>::T) / 64);   // 16-byte pieces per quarter row
                const uint4 *srow = reinterpret_cast<const uint4 *>(reinterpret_cast<const unsigned char *>(src) +
                                                                    (row0 + (size_t)r * kD) * sizeof(typename Elem<DT>::T)) + qt * kVec;
                uint4 *drow = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(side ? a.ch.exact_v : a.ch.exact_k) +
                                                        (size_t)s * kD * sizeof(typename Elem<DT>::T)) + qt * kVec;
#pragma unroll
                for (int k = 0; k < kVec; ++k) drow[k] = srow[k];
                if (qt == 0 && side == 0) a.ch.exact_pos[s] = t_abs;
            } else if (cc == 0 && side == 0 && qt == 0) {
                a.ch.evicted_pos[s] = t_abs;
            }
        }
        group_sync(gid);
    }
}

// ----------------------------------------------------------------------------------------------
// Quantise kernel on the fifth-generation tensor cores (16-bit caches).
//
// Same arithmetic and the same emitted bytes as quantize_kernel above, another mapping.  A CTA (256 threads, two per
// SM) takes whole plan tiles of 128 tokens of one side (keys or values); two threads own a token row, 64 coordinates
// each, and keep them in registers from the global load to the normalisation:
//   norm     the ascending fp32 FMA chain of squares runs over the first thread's half, then over the second's
//            (the partial sum is handed over through shared memory), IEEE square root;
//   divide   x / (norm + 1e-10) as fp32(fp64(x) * fp64(1 / den)) (see quantize_kernel), split into fp16 high and
//            low limbs, written straight into tensor memory (tcgen05.st: a thread's row is its tensor-memory lane) as
//            the A operand;
//   rotate   y = x Pi^T as three tcgen05 products (high x high, high x low, low x high; M 128, N 128, K 128 in
//            eight steps each) with the limbs of Pi in shared memory (K-major, 128-byte swizzle), fp32 accumulator in
//            tensor memory: 24 tensor-core instructions per 128 tokens instead of 3 072 mma.sync plus their
//            ldmatrix traffic;
//   decide   the thread reads its 64 accumulator columns (tcgen05.ld), takes the fp16 decision against the midpoints
//            and packs its half row; coordinates inside the margin of a midpoint are queued;
//   exact    queued coordinates are recomputed with the fp32 chain and the exact rule (the row is re-read from
//            global memory, which just delivered it) and patched into the packed row; 8-bit rows, whose every
//            coordinate is exact work, go to global memory directly;
//   copy-out packed rows, norms, positions; exact-class rows from the registers that still hold them.
// The error of the tensor-core rotation against the chain obeys the bound at kTcMarginBits (three limb products,
// fp32 accumulation of 24 steps), so the margin and with it the emitted codes are the same.
// ----------------------------------------------------------------------------------------------
namespace umma {

constexpr int kThreads = 256;
constexpr int kUQueueCap = 1024;
constexpr int kPkLd = 84;                        // bytes per packed row in shared memory (64 used by a 4-bit row); 21 words:
                                                 // the 32 rows of a warp fall into 32 different banks
constexpr int kPiTileBytes = kD * kD * 2;        // one limb of the rotation, fp16
constexpr unsigned kPolls = 1u << 12;
constexpr unsigned kSuspendNs = 1000000u;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// K-major, 128-byte swizzle, 1024 bytes between 8-row groups, descriptor version 1
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// fp32 accumulator, fp16 operands, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((128u >> 4) << 24);
// D (tensor memory) (+)= A (tensor memory: lane = row, one 32-bit column = two K elements) . B (shared memory)
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d), "r"(a), "l"(bdesc), "r"(kIdesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, unsigned parity) {
    for (unsigned it = 0; it < kPolls; ++it) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(bar), "r"(parity), "r"(kSuspendNs) : "memory");
        if (ok) return true;
    }
    return false;
}
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

template <int DT>
__device__ __forceinline__ float2 unpack16(uint32_t w) {
    if constexpr (DT == kF16) return __half22float2(*reinterpret_cast<const __half2 *>(&w));
    else return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w));
}

constexpr size_t kSmemBytes = 2 * (size_t)kPiTileBytes + (size_t)kTile * kPkLd + 4 * 256 * sizeof(float) + kTile * sizeof(float) * 2 +
                              kTile * sizeof(double) + (2 * kTile + 4 * kNumClasses + 16) * sizeof(int) + (size_t)kUQueueCap * 2 + 1024;

}  // namespace umma

template <int DT>
__global__ void __launch_bounds__(umma::kThreads, 2) quantize_umma_kernel(const QuantArgs a, unsigned *status) {
    using namespace umma;
    extern __shared__ __align__(1024) unsigned char smem_umma[];
    __shared__ __align__(8) uint64_t mma_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ LevelConst lc[3];
    unsigned char *Ph = smem_umma;                                  // rotation, fp16 high limbs, [2 blocks][128 rows][128 bytes] swizzled
    unsigned char *Pl = Ph + kPiTileBytes;                         // low limbs
    unsigned char *PK = Pl + kPiTileBytes;                         // [128][kPkLd] packed rows
    float *cb = reinterpret_cast<float *>(PK + kTile * kPkLd);     // [4][256]
    float *nrm = cb + 4 * 256;                                     // [128]
    float *part = nrm + kTile;                                     // [128] chain value after the first half
    double *rinv = reinterpret_cast<double *>(part + kTile);       // [128]
    int *cls = reinterpret_cast<int *>(rinv + kTile);              // [128]
    int *slot = cls + kTile;                                       // [128]
    int *wcnt = slot + kTile;                                      // [4][6]
    int *tbase = wcnt + 4 * kNumClasses;                           // [8]
    int *flags = tbase + 8;                                        // [0] any quantised row, [1] queue length
    uint16_t *queue = reinterpret_cast<uint16_t *>(flags + 8);     // [kUQueueCap]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = (warp & 3) * 32 + lane, half = warp >> 2;      // token row of the tile, coordinate half
    const int B = a.ch.B, H = a.ch.H, T = a.ch.T, BH = B * H;
    const int side = blockIdx.x & 1;
    const unsigned char *src = reinterpret_cast<const unsigned char *>(side ? a.V : a.K);
    const float *pi = side ? a.pi_v : a.pi_k;

    // ---- rotation limbs: element (j, i) of a limb sits in block i / 64 at j * 128 + ((i % 64) / 8 ^ (j % 8)) * 16 + (i % 8) * 2
    for (int g = tid; g < kD * kD / 8; g += kThreads) {
        const int j = g >> 4, c = g & 15;                          // row, 16-byte chunk (eight coordinates)
        const float4 f0 = *reinterpret_cast<const float4 *>(pi + j * kD + 8 * c), f1 = *reinterpret_cast<const float4 *>(pi + j * kD + 8 * c + 4);
        const float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __half2 h = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
            const float2 bk = __half22float2(h);
            hw[k] = h2u(h);
            lw[k] = h2u(__floats2half2_rn(f[2 * k] - bk.x, f[2 * k + 1] - bk.y));
        }
        const size_t off = (size_t)(c >> 3) * (kD * 128) + (size_t)j * 128 + (size_t)(((c & 7) ^ (j & 7)) * 16);
        *reinterpret_cast<uint4 *>(Ph + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *reinterpret_cast<uint4 *>(Pl + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
    for (int g = tid; g < 4 * 256; g += kThreads) cb[g] = a.codebooks[g];
    if (tid < 3 * 8) {
        const int li = tid >> 3, j = tid & 7, half_k = 1 << (li + 1);   // K/2 for 2, 3, 4 bits
        const float *cbl = a.codebooks + li * 256;
        if (j < 7) {
            __half m = __ushort_as_half((unsigned short)0x7c00);        // +inf: never exceeded, never near
            if (j + 1 < half_k) m = __float2half_rn(0.5f * (cbl[half_k + j] + cbl[half_k + j + 1]));
            lc[li].mid[j] = h2u(__half2half2(m));
        } else {
            lc[li].base = h2u(__half2half2(__float2half_rn(512.0f + (float)half_k - 0.5f)));
        }
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&mma_bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    proxy_fence();            // the limbs were written by ordinary stores and are read by the tensor cores
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t t_ah = t_lane + half * 32, t_al = t_lane + 64 + half * 32, t_d = t_lane + 128 + half * 64;

    const long long n_work = (long long)BH * a.ntiles;
    const long long w_step = gridDim.x >> 1;
    unsigned n_mma = 0;          // products committed so far (parity of the barrier)
    bool dead = false;
    // this thread's 64 coordinates of the current tile, kept as 32 packed words; the next tile's are fetched as soon as
    // the current ones have been normalised, so that their latency runs under the decision and the recomputation
    uint32_t raw[32];
    auto load_raw = [&](long long w2) {
        const int bh2 = (int)(w2 / a.ntiles), tl2 = (int)(w2 % a.ntiles);
        const bool live2 = w2 < n_work && tl2 * kTile + row < T;
        const uint4 *rp = reinterpret_cast<const uint4 *>(src + (((size_t)bh2 * T + (size_t)tl2 * kTile + row) * kD + 64 * half) * 2);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint4 v = live2 ? __ldg(rp + u) : make_uint4(0u, 0u, 0u, 0u);
            raw[4 * u] = v.x; raw[4 * u + 1] = v.y; raw[4 * u + 2] = v.z; raw[4 * u + 3] = v.w;
        }
    };
    load_raw(blockIdx.x >> 1);
    for (long long w = blockIdx.x >> 1; w < n_work; w += w_step) {
        const int bh = (int)(w / a.ntiles), tile = (int)(w % a.ntiles);
        const int t0 = tile * kTile;
        if (tid == 0) { flags[0] = 0; flags[1] = 0; }
        // ---- classes and slots of the plan tile (the slot of a token counts the tokens before it)
        int c = -1, rank = 0;
        if (tid < kTile) {
            if (t0 + tid < T) c = class_of_bits(a.bits[(size_t)bh * T + t0 + tid]);
#pragma unroll
            for (int cc = 0; cc < kNumClasses; ++cc) {
                unsigned m = __ballot_sync(0xffffffffu, c == cc);
                if (c == cc) rank = __popc(m & ((1u << lane) - 1u));
                if (lane == 0) wcnt[warp * kNumClasses + cc] = __popc(m);
            }
            if (tid < kNumClasses) tbase[tid] = a.ch.seg_start[tid * BH + bh] + a.tile_base[((size_t)bh * a.ntiles + tile) * kNumClasses + tid];
        }
        // ---- norm chain, first half of every row
        float acc = 0.0f;
        if (half == 0) {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
                const float2 f = unpack16<DT>(raw[k]);
                acc = fmaf(f.x, f.x, acc);
                acc = fmaf(f.y, f.y, acc);
            }
            part[row] = acc;
        }
        __syncthreads();
        if (tid < kTile) {
            int s = -1;
            if (c >= 0) {
                s = tbase[c] + rank;
                for (int ww = 0; ww < warp; ++ww) s += wcnt[ww * kNumClasses + c];
                if (c >= 1 && c <= 4) flags[0] = 1;
            }
            cls[tid] = c;
            slot[tid] = s;
        }
        if (half == 1) {
            acc = part[row];
#pragma unroll
            for (int k = 0; k < 32; ++k) {
                const float2 f = unpack16<DT>(raw[k]);
                acc = fmaf(f.x, f.x, acc);
                acc = fmaf(f.y, f.y, acc);
            }
            const float nr = __fsqrt_rn(acc);
            nrm[row] = nr;
            rinv[row] = 1.0 / (double)__fadd_rn(nr, 1e-10f);
        }
        __syncthreads();
        const bool any_q = flags[0] != 0;
        const int cc = cls[row];
        if (cc == 5) {   // exact class: the row goes out as it came in
            const int s = slot[row];
            uint4 *drow = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(side ? a.ch.exact_v : a.ch.exact_k) + ((size_t)s * kD + 64 * half) * 2);
#pragma unroll
            for (int u = 0; u < 8; ++u) drow[u] = make_uint4(raw[4 * u], raw[4 * u + 1], raw[4 * u + 2], raw[4 * u + 3]);
        }
        if (any_q) {
            // ---- normalise, split into limbs, A operand into tensor memory
            {
                const double ri = rinv[row];
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    const float2 f = unpack16<DT>(raw[k]);
                    const float x0 = __double2float_rn(__dmul_rn((double)f.x, ri)), x1 = __double2float_rn(__dmul_rn((double)f.y, ri));
                    const __half2 h = __floats2half2_rn(x0, x1);
                    const float2 bk = __half22float2(h);
                    hi[k] = h2u(h);
                    lo[k] = h2u(__floats2half2_rn(x0 - bk.x, x1 - bk.y));
                }
                tmem_st32(t_ah, hi);
                tmem_st32(t_al, lo);
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            load_raw(w + w_step);
            tc_fence_before();
            __syncthreads();
            if (warp == 0 && !dead) {
                tc_fence_after();
                uint32_t elected;
                asm volatile("{\n.reg .pred P1;\nelect.sync _|P1, 0xffffffff;\nselp.u32 %0, 1, 0, P1;\n}\n" : "=r"(elected));
                if (elected) {
                    const uint32_t d = tmem + 128, ah = tmem, al = tmem + 64;
                    const uint32_t ph = smem_u32(Ph), pl = smem_u32(Pl);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t bo = (ks >> 2) * (kD * 128) + (ks & 3) * 32;
                        mma_ts(d, al + ks * 8, smem_desc(ph + bo), ks ? 1u : 0u);
                        mma_ts(d, ah + ks * 8, smem_desc(pl + bo), 1u);
                        mma_ts(d, ah + ks * 8, smem_desc(ph + bo), 1u);
                    }
                    mma_commit(smem_u32(&mma_bar));
                }
                __syncwarp();
            }
            if (!dead && !mbar_wait(smem_u32(&mma_bar), n_mma & 1)) {
                dead = true;
                atomicExch(status, 1u);
            }
            n_mma += 1;
            tc_fence_after();
            // ---- fp16 decision and packing of this thread's 64 coordinates (eight groups of eight).  The
            //      tensor-memory loads are warp-wide instructions: every thread takes them, whatever its row's class.
            const bool quant_row = cc >= 1 && cc <= 3;
            const LevelConst &L = lc[quant_row ? cc - 1 : 0];
            uint32_t mid[7];
#pragma unroll
            for (int j = 0; j < 7; ++j) mid[j] = L.mid[j];
            const uint32_t base = L.base;
            const int b = quant_row ? cc + 1 : 2;              // bits per code
            unsigned char *dst = PK + row * kPkLd + half * 8 * b;
#pragma unroll 1
            for (int cbk = 0; cbk < 2; ++cbk) {
                uint32_t v[32];
                tmem_ld32(t_d + cbk * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (quant_row) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {              // eight coordinates -> b bytes
                        uint32_t word = 0, bad = 0;
#pragma unroll
                        for (int nb = 0; nb < 4; ++nb) {
                            const uint32_t y2 = h2u(__floats2half2_rn(__uint_as_float(v[8 * q + 2 * nb]), __uint_as_float(v[8 * q + 2 * nb + 1])));
                            uint32_t ok;
                            const uint32_t cf = cc == 3 ? decide_pair<7>(y2, mid, base, ok) : decide_pair<3>(y2, mid, base, ok);
                            const uint32_t field = ((cf >> 1) & 15u) | (((cf >> 17) & 15u) << b);
                            word |= field << (2 * b * nb);
                            if ((ok & 0xffffu) != 0x3c00u) bad |= 1u << (2 * nb);
                            if ((ok >> 16) != 0x3c00u) bad |= 2u << (2 * nb);
                        }
                        unsigned char *dq = dst + (cbk * 4 + q) * b;
                        if (b == 2) *reinterpret_cast<uint16_t *>(dq) = (uint16_t)word;
                        else if (b == 4) *reinterpret_cast<uint32_t *>(dq) = word;
                        else { dq[0] = (unsigned char)word; dq[1] = (unsigned char)(word >> 8); dq[2] = (unsigned char)(word >> 16); }
                        while (bad) {
                            const int c8 = __ffs(bad) - 1;
                            bad &= bad - 1;
                            const int qi = atomicAdd(&flags[1], 1);
                            if (qi < kUQueueCap) queue[qi] = (uint16_t)((row << 7) | (64 * half + 32 * cbk + 8 * q + c8));
                        }
                    }
                }
            }
            if (cc == 4) {   // 8 bits: the centroid spacing is within the margin, every coordinate is exact work
                for (int c8 = 0; c8 < 64; ++c8) {
                    const int qi = atomicAdd(&flags[1], 1);
                    if (qi < kUQueueCap) queue[qi] = (uint16_t)((row << 7) | (64 * half + c8));
                }
            }
            tc_fence_before();
            __syncthreads();
            // ---- exact recomputation of the queued coordinates: ascending fp32 FMA chain over the re-read row.  Four
            //      lanes share a coordinate: each fetches and normalises a quarter of the row (the conversions are the
            //      bulk of the work and run side by side), then the chain walks through the quarters in ascending
            //      order, its running value handed from lane to lane -- the same sequence of fused multiply-adds as
            //      one thread would execute.
            const int qn = flags[1];
            const bool redo_all = qn > kUQueueCap;   // queue overflow: every coordinate of the tile is exact work
            const int n_fix = redo_all ? kTile * kD : qn;
            const int sub = lane & 3;
            for (int e0 = 0; e0 < n_fix; e0 += kThreads / 4) {     // same trip count for every thread of the CTA
                const int e = e0 + (tid >> 2);
                int r = 0, col = 0, li = -1;
                if (e < n_fix) {
                    r = redo_all ? (e >> 7) : (queue[e] >> 7);
                    col = redo_all ? (e & 127) : (queue[e] & 127);
                    li = cls[r] - 1;
                }
                const bool work = li >= 0 && li <= 3;
                float xn[32], pv[32];
                if (work) {
                    const uint4 *xr = reinterpret_cast<const uint4 *>(src + (((size_t)bh * T + t0 + r) * kD + 32 * sub) * 2);
                    const float4 *pr = reinterpret_cast<const float4 *>(pi + col * kD + 32 * sub);
                    uint4 xv[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) xv[u] = __ldg(xr + u);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float4 p = __ldg(pr + u);
                        pv[4 * u] = p.x; pv[4 * u + 1] = p.y; pv[4 * u + 2] = p.z; pv[4 * u + 3] = p.w;
                    }
                    const double ri = rinv[r];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t xw[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float2 f = unpack16<DT>(xw[k]);
                            xn[8 * u + 2 * k] = __double2float_rn(__dmul_rn((double)f.x, ri));
                            xn[8 * u + 2 * k + 1] = __double2float_rn(__dmul_rn((double)f.y, ri));
                        }
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 32; ++k) { xn[k] = 0.0f; pv[k] = 0.0f; }
                }
                float y = 0.0f;
#pragma unroll
                for (int st = 0; st < 4; ++st) {
                    if (sub == st) {
#pragma unroll
                        for (int k = 0; k < 32; ++k) y = fmaf(xn[k], pv[k], y);
                    }
                    y = __shfl_sync(0xffffffffu, y, (lane & ~3) | st);   // the next quarter continues from here
                }
                if (work && sub == 0) {
                    const int code = nearest_centroid(y, cb + li * 256, 1 << bits_of_qlevel(li));
                    if (li == 3) {
                        uint8_t *rows8 = side ? a.ch.v_codes[3] : a.ch.k_codes[3];
                        rows8[(size_t)slot[r] * 128 + col] = (uint8_t)code;
                    } else {
                        patch_code(reinterpret_cast<uint32_t *>(PK + r * kPkLd), qbits(li), col, (uint32_t)code);
                    }
                }
            }
            __syncthreads();
        } else {
            load_raw(w + w_step);
        }
        // ---- copy-out: this thread's half row
        {
            const int s = slot[row];
            const int t_abs = a.ch.t_offset + t0 + row;
            if (cc >= 1 && cc <= 3) {
                const int li = cc - 1, nw = 2 * qbits(li);       // words per half row
                uint8_t *rows = side ? a.v_scratch[li] : a.k_scratch[li];
                uint32_t *dst = reinterpret_cast<uint32_t *>(rows + (size_t)s * 16 * qbits(li)) + half * nw;
                const uint32_t *srcw = reinterpret_cast<const uint32_t *>(PK + row * kPkLd) + half * nw;
                for (int k = 0; k < nw; ++k) dst[k] = srcw[k];
            }
            if (cc >= 1 && cc <= 4 && half == 0) {
                const int li = cc - 1;
                (side ? a.ch.v_norm[li] : a.ch.k_norm[li])[s] = nrm[row];
                if (side == 0) a.ch.pos[li][s] = t_abs;
            } else if (cc == 5) {
                if (half == 0 && side == 0) a.ch.exact_pos[s] = t_abs;
            } else if (cc == 0 && side == 0 && half == 0) {
                a.ch.evicted_pos[s] = t_abs;
            }
        }
        __syncthreads();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(256u) : "memory");
}

// zero the padding slots between a segment's last token and the next 16-slot boundary
template <int DT>
__global__ void fill_padding_kernel(const odmkv_chunk ch, uint8_t *k_scratch0, uint8_t *k_scratch1, uint8_t *k_scratch2,
                                    uint8_t *v_scratch0, uint8_t *v_scratch1, uint8_t *v_scratch2) {
    uint8_t *k_scratch[3] = {k_scratch0, k_scratch1, k_scratch2};
    uint8_t *v_scratch[3] = {v_scratch0, v_scratch1, v_scratch2};
    __shared__ uint8_t zero_row[kD];
    if (threadIdx.x < kD) zero_row[threadIdx.x] = 0;
    __syncthreads();
    const int BH = ch.B * ch.H;
    const int bh = blockIdx.x, c = blockIdx.y;
    const int cnt = ch.seg_count[c * BH + bh];
    const int start = ch.seg_start[c * BH + bh];
    const int pad_end = ((cnt + kSegAlign - 1) / kSegAlign) * kSegAlign;
    for (int k = cnt + (threadIdx.x >> 5); k < pad_end; k += blockDim.x >> 5) {
        const int s = start + k, lane = threadIdx.x & 31;
        if (c == 0) {
            if (lane == 0) ch.evicted_pos[s] = -1;
        } else if (c == 5) {
            using T = typename Elem<DT>::T;
            T *kr = reinterpret_cast<T *>(ch.exact_k) + (size_t)s * kD;
            T *vr = reinterpret_cast<T *>(ch.exact_v) + (size_t)s * kD;
            for (int i = lane; i < kD; i += 32) {
                kr[i] = Elem<DT>::from_f32(0.f);
                vr[i] = Elem<DT>::from_f32(0.f);
            }
            if (lane == 0) ch.exact_pos[s] = -1;
        } else {
            const int li = c - 1;
            store_linear_codes(zero_row, li, li == 3 ? ch.k_codes[3] : k_scratch[li], s, lane);
            store_linear_codes(zero_row, li, li == 3 ? ch.v_codes[3] : v_scratch[li], s, lane);
            if (lane == 0) {
                ch.k_norm[li][s] = 0.f;
                ch.v_norm[li][s] = 0.f;
                ch.pos[li][s] = -1;
            }
        }
    }
}

// NB bits (at most 32) at a compile-time bit offset of a little-endian word array held in registers
template <int NB>
__device__ __forceinline__ uint32_t extract_bits(const uint32_t *w, int off) {
    const int wi = off >> 5, sh = off & 31;
    const uint32_t v = (sh + NB <= 32) ? (w[wi] >> sh) : __funnelshift_r(w[wi], w[wi + 1], sh);
    return NB == 32 ? v : (v & ((NB == 32 ? 0u : (1u << (NB & 31))) - 1u));
}
// OR a field of NB bits into a zero-initialised word array at a compile-time bit offset
template <int NB>
__device__ __forceinline__ void insert_bits(uint32_t *out, int off, uint32_t field) {
    const int wi = off >> 5, sh = off & 31;
    out[wi] |= field << sh;
    if (sh + NB > 32) out[wi + 1] |= field >> (32 - sh);
}

// re-tile the codes of one 2/3/4-bit bank: linear scratch rows -> tensor-core tile layout
// (one warp per tile of 16 slots; lane (g, t) assembles its own 8*b bytes; KEYS selects the field map).
// A lane's source bits are few whole words, so it loads them once and moves the fields between registers:
//   keys:   the 32 coordinates 32 t .. 32 t + 31 of slots g and g + 8 are b consecutive words of either row; field
//           4 s + 2 odd + hi of the output is pair 2 s + odd of slot g + 8 hi;
//   values: coordinate 16 m + g + 8 a of a row sits at bit b g of its group 2 m + a of 8 b bits, so a lane shifts
//           every group of the four rows 2 t, 2 t + 1, 2 t + 8, 2 t + 9 by the same amount.
template <int B, bool KEYS>
__global__ void retile_kernel(const uint8_t *__restrict__ rows, uint8_t *__restrict__ bank, int ntiles) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    constexpr uint32_t kMask = (1u << B) - 1u;
    for (int tile = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); tile < ntiles; tile += gridDim.x * (blockDim.x >> 5)) {
        uint32_t out[2 * B];
#pragma unroll
        for (int w = 0; w < 2 * B; ++w) out[w] = 0;
        const uint32_t *tile_rows = reinterpret_cast<const uint32_t *>(rows + (size_t)tile * 16 * 16 * B);   // 4 B words per row
        if (KEYS) {
            uint32_t c[2][B];
#pragma unroll
            for (int hi = 0; hi < 2; ++hi)
#pragma unroll
                for (int w = 0; w < B; ++w) c[hi][w] = __ldg(tile_rows + (g + 8 * hi) * 4 * B + B * t + w);
#pragma unroll
            for (int f = 0; f < 32; ++f) {
                const int pair = f >> 1, hi = f & 1;   // pair = 2 s + odd
                insert_bits<2 * B>(out, 2 * B * f, extract_bits<2 * B>(c[hi], 2 * B * pair));
            }
        } else {
            const int sh = B * g;
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {
                uint32_t ra[4 * B], rb[4 * B];
                const uint4 *pa = reinterpret_cast<const uint4 *>(tile_rows + (2 * t + 8 * hi) * 4 * B);
                const uint4 *pb = reinterpret_cast<const uint4 *>(tile_rows + (2 * t + 8 * hi + 1) * 4 * B);
#pragma unroll
                for (int u = 0; u < B; ++u) {
                    const uint4 va = __ldg(pa + u), vb = __ldg(pb + u);
                    ra[4 * u] = va.x; ra[4 * u + 1] = va.y; ra[4 * u + 2] = va.z; ra[4 * u + 3] = va.w;
                    rb[4 * u] = vb.x; rb[4 * u + 1] = vb.y; rb[4 * u + 2] = vb.z; rb[4 * u + 3] = vb.w;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {            // j = 2 m + a
                    const uint32_t ga = extract_bits<8 * B>(ra, 8 * B * j), gb = extract_bits<8 * B>(rb, 8 * B * j);
                    const uint32_t field = ((ga >> sh) & kMask) | (((gb >> sh) & kMask) << B);
                    insert_bits<2 * B>(out, 2 * B * (4 * (j >> 1) + 2 * hi + (j & 1)), field);
                }
            }
        }
        uint32_t *dst = reinterpret_cast<uint32_t *>(bank + (size_t)tile * 256 * B + (size_t)lane * 8 * B);
#pragma unroll
        for (int w = 0; w < 2 * B; ++w) dst[w] = out[w];
    }
}

// nearest centroid + pack of given rotated coordinates; one warp per row
__global__ void encode_pack_kernel(const float *__restrict__ y, long long n, int li, const float *__restrict__ codebook,
                                   uint8_t *__restrict__ out) {
    __shared__ float cb[256];
    __shared__ uint8_t stage[8][kD];
    const int k = 1 << bits_of_qlevel(li);
    for (int i = threadIdx.x; i < k; i += blockDim.x) cb[i] = codebook[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (long long r = (long long)blockIdx.x * 8 + warp; r < n; r += (long long)gridDim.x * 8) {
#pragma unroll
        for (int q = 0; q < 4; ++q) stage[warp][lane + 32 * q] = (uint8_t)nearest_centroid(y[r * kD + lane + 32 * q], cb, k);
        __syncwarp();
        store_linear_codes(stage[warp], li, out, r, lane);
        __syncwarp();
    }
}

// ----------------------------------------------------------------------------------------------
// Dequantise
// ----------------------------------------------------------------------------------------------
struct DequantArgs {
    odmkv_chunk ch;
    const float *pi_k;
    const float *pi_v;
    const float *codebooks;
    void *K_out;
    void *V_out;
    int T_dense;
    int tiles_before[5];  // prefix of tile counts per quantised level
};

__device__ inline int bank_end(const odmkv_chunk &ch, int c) {
    const int BH = ch.B * ch.H;
    int cnt = ch.seg_count[c * BH + BH - 1];
    return ch.seg_start[c * BH + BH - 1] + ((cnt + kSegAlign - 1) / kSegAlign) * kSegAlign;
}

// largest bh with seg_start[bh] <= s
__device__ inline int find_segment(const int32_t *__restrict__ seg_start, int BH, int s) {
    int lo = 0, hi = BH;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (seg_start[mid] <= s) lo = mid; else hi = mid;
    }
    return lo;
}

template <int ODT>
__global__ void __launch_bounds__(256, 1) dequant_kernel(const DequantArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *PkT = reinterpret_cast<float *>(smem_raw);  // PkT[j][i] = pi_k[i][j]
    float *PvT = PkT + kD * kLd;
    float *Xs = PvT + kD * kLd;
    float *cb = Xs + kD * kLd;
    float *nrm = cb + 4 * 256;
    long long *dst_row = reinterpret_cast<long long *>(nrm + kTile);  // [128] dense row index or -1

    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;
    const int BH = a.ch.B * a.ch.H;
    for (int g = tid; g < kD * kD; g += 256) {
        int i = g >> 7, j = g & 127;
        PkT[j * kLd + i] = a.pi_k[g];
        PvT[j * kLd + i] = a.pi_v[g];
    }
    for (int g = tid; g < 4 * 256; g += 256) cb[g] = a.codebooks[g];
    __syncthreads();

    const int n_work = a.tiles_before[4];
    for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
        int li = 0;
        while (li < 3 && w >= a.tiles_before[li + 1]) ++li;
        const int c = li + 1;
        const int s0 = (w - a.tiles_before[li]) * kTile;
        const int end = bank_end(a.ch, c);
        if (s0 >= end) continue;  // uniform across the block
        if (tid < kTile) {
            int s = s0 + tid;
            long long row = -1;
            if (s < end) {
                const int t = a.ch.pos[li][s];
                const int bh = find_segment(a.ch.seg_start + c * BH, BH, s);
                // a slot counts only while it lies inside its segment's current length (truncation shortens
                // segments without touching the banks) and its position fits the dense tensor
                if (t >= 0 && t < a.T_dense && s - a.ch.seg_start[c * BH + bh] < a.ch.seg_count[c * BH + bh])
                    row = (long long)bh * a.T_dense + t;
            }
            dst_row[tid] = row;
        }
        for (int side = 0; side < 2; ++side) {
            const uint8_t *codes = side ? a.ch.v_codes[li] : a.ch.k_codes[li];
            const float *norms = side ? a.ch.v_norm[li] : a.ch.k_norm[li];
            const float *Ps = side ? PvT : PkT;
            __syncthreads();
            {   // centroid gather: two threads per row
                int r = tid >> 1, half = tid & 1, s = s0 + r;
                bool ok = s < end;
                const float *cbl = cb + li * 256;
                for (int i = half * 64; i < half * 64 + 64; ++i) {
                    float v = 0.f;
                    if (ok) v = cbl[side ? v_code(codes, li, s, i) : k_code(codes, li, s, i)];
                    Xs[r * kLd + i] = v;
                }
                if (half == 0) nrm[r] = ok ? norms[s] : 0.f;
            }
            __syncthreads();
            float acc[8][8];
            tile_product(Xs, Ps, ty, tx, acc);
            __syncthreads();
#pragma unroll
            for (int aa = 0; aa < 8; ++aa) {
                int r = ty + 16 * aa;
                float nn = nrm[r];
#pragma unroll
                for (int bb = 0; bb < 8; ++bb) Xs[r * kLd + tx + 16 * bb] = __fmul_rn(acc[aa][bb], nn);
            }
            __syncthreads();
            void *out = side ? a.V_out : a.K_out;
            for (int g = tid; g < kTile * kD / 4; g += 256) {
                int r = g >> 5, i4 = g & 31;
                long long row = dst_row[r];
                if (row >= 0) store4<ODT>(out, (size_t)row * kD + 4 * i4, *reinterpret_cast<const float4 *>(Xs + r * kLd + 4 * i4));
            }
        }
        __syncthreads();
    }
}

// scatter the exact bank into the dense tensors; one warp per slot
template <int IDT, int ODT>
__global__ void scatter_exact_kernel(const odmkv_chunk ch, void *K_out, void *V_out, int T_dense) {
    const int BH = ch.B * ch.H;
    const int end = bank_end(ch, 5);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int s = blockIdx.x * (blockDim.x >> 5) + warp; s < end; s += gridDim.x * (blockDim.x >> 5)) {
        int t = ch.exact_pos[s];
        if (t < 0 || t >= T_dense) continue;
        int bh = find_segment(ch.seg_start + 5 * BH, BH, s);
        if (s - ch.seg_start[5 * BH + bh] >= ch.seg_count[5 * BH + bh]) continue;
        size_t dst = ((size_t)bh * T_dense + t) * kD + 4 * lane;
        store4<ODT>(K_out, dst, load4<IDT>(ch.exact_k, (size_t)s * kD + 4 * lane));
        store4<ODT>(V_out, dst, load4<IDT>(ch.exact_v, (size_t)s * kD + 4 * lane));
    }
}

// ----------------------------------------------------------------------------------------------
// Export to the reference bank layout
// ----------------------------------------------------------------------------------------------
__global__ void export_bank_kernel(const odmkv_chunk ch, int c, const int32_t *__restrict__ row_start,
                                   uint8_t *__restrict__ ik, uint8_t *__restrict__ iv, float *__restrict__ nk,
                                   float *__restrict__ nv, int64_t *__restrict__ positions) {
    const int BH = ch.B * ch.H, bh = blockIdx.x, li = c - 1;
    const int cnt = ch.seg_count[c * BH + bh], s0 = ch.seg_start[c * BH + bh], r0 = row_start[bh];
    const int rb = ref_code_bytes(li);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int k = warp; k < cnt; k += blockDim.x >> 5) {
        const size_t s = (size_t)s0 + k, r = (size_t)r0 + k;
        for (int side = 0; side < 2; ++side) {
            const uint8_t *bank = side ? ch.v_codes[li] : ch.k_codes[li];
            uint8_t *dst = (side ? iv : ik) + r * rb;
            for (int j = lane; j < rb; j += 32) {
                uint32_t out = 0;
                if (li == 0) {
                    for (int e = 0; e < 4; ++e) out |= (uint32_t)(side ? v_code(bank, li, s, 4 * j + e) : k_code(bank, li, s, 4 * j + e)) << (2 * e);
                } else if (li == 3) {
                    out = side ? v_code(bank, li, s, j) : k_code(bank, li, s, j);
                } else {
                    for (int e = 0; e < 2; ++e) out |= (uint32_t)(side ? v_code(bank, li, s, 2 * j + e) : k_code(bank, li, s, 2 * j + e)) << (4 * e);
                }
                dst[j] = (uint8_t)out;
            }
        }
        if (lane == 0) {
            nk[r] = ch.k_norm[li][s];
            nv[r] = ch.v_norm[li][s];
            positions[3 * r + 0] = bh / ch.H;
            positions[3 * r + 1] = bh % ch.H;
            positions[3 * r + 2] = ch.pos[li][s];
        }
    }
}

__global__ void export_positions_kernel(const odmkv_chunk ch, int c, const int32_t *__restrict__ row_start,
                                        int64_t *__restrict__ positions) {
    const int BH = ch.B * ch.H, bh = blockIdx.x;
    const int cnt = ch.seg_count[c * BH + bh], s0 = ch.seg_start[c * BH + bh], r0 = row_start[bh];
    const int32_t *pos = c == 0 ? ch.evicted_pos : ch.exact_pos;
    for (int k = threadIdx.x; k < cnt; k += blockDim.x) {
        size_t r = (size_t)r0 + k;
        positions[3 * r + 0] = bh / ch.H;
        positions[3 * r + 1] = bh % ch.H;
        positions[3 * r + 2] = pos[s0 + k];
    }
}

// ----------------------------------------------------------------------------------------------
// Compaction: several chunks -> one (same slot order inside every (b, h) segment: chunk after chunk)
// ----------------------------------------------------------------------------------------------
struct CompactArgs {
    odmkv_chunk src[kMaxChunks];
    odmkv_chunk dst;
    const int32_t *dst_off;     // [n_src, 6, B*H]: first destination slot of chunk i's tokens inside the destination segment
    uint8_t *k_scratch[3];      // linear-layout codes of the destination's 2/3/4-bit banks before re-tiling
    uint8_t *v_scratch[3];
    int n_src;
};

// grid (B*H, n_src, 6 classes); a warp moves one slot at a time
template <int DT>
__global__ void compact_gather_kernel(const CompactArgs a) {
    __shared__ uint8_t stage[8][kD];
    const int bh = blockIdx.x, i = blockIdx.y, c = blockIdx.z;
    const odmkv_chunk &src = a.src[i];
    const int BH = a.dst.B * a.dst.H;
    const int cnt = src.seg_count[c * BH + bh];
    if (cnt == 0) return;
    const int s0 = src.seg_start[c * BH + bh];
    const int d0 = a.dst.seg_start[c * BH + bh] + a.dst_off[((size_t)i * kNumClasses + c) * BH + bh];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int k = warp; k < cnt; k += blockDim.x >> 5) {
        const long long s = (long long)s0 + k, d = (long long)d0 + k;
        if (c == 0) {
            if (lane == 0) a.dst.evicted_pos[d] = src.evicted_pos[s];
        } else if (c == 5) {
            using T = typename Elem<DT>::T;
            const T *ks = reinterpret_cast<const T *>(src.exact_k) + (size_t)s * kD, *vs = reinterpret_cast<const T *>(src.exact_v) + (size_t)s * kD;
            T *kd = reinterpret_cast<T *>(a.dst.exact_k) + (size_t)d * kD, *vd = reinterpret_cast<T *>(a.dst.exact_v) + (size_t)d * kD;
            for (int e = lane; e < kD; e += 32) { kd[e] = ks[e]; vd[e] = vs[e]; }
            if (lane == 0) a.dst.exact_pos[d] = src.exact_pos[s];
        } else {
            const int li = c - 1;
            for (int side = 0; side < 2; ++side) {
                const uint8_t *bank = side ? src.v_codes[li] : src.k_codes[li];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int dim = 4 * lane + q;
                    stage[warp][dim] = (uint8_t)(side ? v_code(bank, li, s, dim) : k_code(bank, li, s, dim));
                }
                __syncwarp();
                uint8_t *rows = li == 3 ? (side ? a.dst.v_codes[3] : a.dst.k_codes[3]) : (side ? a.v_scratch[li] : a.k_scratch[li]);
                store_linear_codes(stage[warp], li, rows, d, lane);
                __syncwarp();
            }
            if (lane == 0) {
                a.dst.k_norm[li][d] = src.k_norm[li][s];
                a.dst.v_norm[li][d] = src.v_norm[li][s];
                a.dst.pos[li][d] = src.pos[li][s];
            }
        }
    }
}

static int num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

constexpr size_t kDequantSmem = (size_t)(3 * kD * kLd + 4 * 256 + kTile) * sizeof(float) + kTile * sizeof(long long);

}  // namespace odmkv

using namespace odmkv;

extern "C" {

size_t odmkv_pack_plan_workspace_bytes(int B, int H, int T) {
    if (B <= 0 || H <= 0 || T <= 0) return 0;
    size_t ntiles = ((size_t)T + kTile - 1) / kTile;
    return 2 * (size_t)B * H * ntiles * kNumClasses * sizeof(int32_t);
}

int odmkv_pack_plan(const int32_t *bits, int B, int H, int T, int32_t *seg_start, int32_t *seg_count,
                    int32_t *totals, void *plan_workspace, size_t plan_workspace_bytes, void *stream) {
    if (!bits || !seg_start || !seg_count || !totals || !plan_workspace) return ODMKV_ERR_ARG;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 65535) return ODMKV_ERR_SHAPE;
    if (plan_workspace_bytes < odmkv_pack_plan_workspace_bytes(B, H, T)) return ODMKV_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int BH = B * H, ntiles = (T + kTile - 1) / kTile;
    int32_t *tile_counts = (int32_t *)plan_workspace;
    int32_t *tile_base = tile_counts + (size_t)BH * ntiles * kNumClasses;
    cudaMemsetAsync(totals, 0, 8 * sizeof(int32_t), st);
    count_tiles_kernel<<<dim3(ntiles, BH), kTile, 0, st>>>(bits, T, ntiles, tile_counts, totals);
    scan_tiles_kernel<<<BH, 32 * kNumClasses, 0, st>>>(tile_counts, ntiles, BH, tile_base, seg_count);
    scan_segs_kernel<<<1, 32 * kNumClasses, 0, st>>>(seg_count, BH, seg_start, totals);
    return launch_status();
}

// status word of the tcgen05 quantise kernel: set to 1 when a bounded wait on the tensor cores expired
__device__ unsigned g_quant_status;
static unsigned *quant_status_ptr() {
    static unsigned *ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_quant_status) != cudaSuccess) return nullptr;
        ptrs[dev] = reinterpret_cast<unsigned *>(p);
    }
    return ptrs[dev];
}

static int check_chunk(const odmkv_chunk *ch) {
    if (!ch || !ch->seg_start || !ch->seg_count) return ODMKV_ERR_ARG;
    if (ch->B <= 0 || ch->H <= 0 || ch->T < 0 || (long long)ch->B * ch->H > 65535) return ODMKV_ERR_SHAPE;
    for (int li = 0; li < ODMKV_NUM_QLEVELS; ++li)
        if (ch->cap[li + 1] > 0 && (!ch->k_codes[li] || !ch->v_codes[li] || !ch->k_norm[li] || !ch->v_norm[li] || !ch->pos[li]))
            return ODMKV_ERR_ARG;
    if (ch->cap[5] > 0 && (!ch->exact_k || !ch->exact_v || !ch->exact_pos)) return ODMKV_ERR_ARG;
    if (ch->cap[0] > 0 && !ch->evicted_pos) return ODMKV_ERR_ARG;
    return ODMKV_OK;
}

size_t odmkv_quantize_workspace_bytes(const int32_t *cap) {
    if (!cap) return 0;
    size_t n = 0;
    for (int li = 0; li < 3; ++li) n += 2 * (((size_t)(cap[li + 1] > 0 ? cap[li + 1] : 0) * 16 * qbits(li) + 255) / 256 * 256);
    return n + 256;
}

// 0 when no tensor-core wait of odmkv_quantize_pack has expired on the current device since the library was loaded
// (synchronises the device); 1 otherwise (the packed codes of that call are invalid); negative on a CUDA error
int odmkv_quantize_status(void) {
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, g_quant_status, sizeof(v)) != cudaSuccess) return -1;
    return v != 0 ? 1 : 0;
}

int odmkv_quantize_pack(const void *K, const void *V, int dtype, const int32_t *bits, const float *pi_k,
                        const float *pi_v, const float *codebooks, const odmkv_chunk *chunk,
                        const void *plan_workspace, void *workspace, size_t workspace_bytes, void *stream) {
    if (!K || !V || !bits || !pi_k || !pi_v || !codebooks || !plan_workspace || !workspace) return ODMKV_ERR_ARG;
    int rc = check_chunk(chunk);
    if (rc) return rc;
    if (((uintptr_t)workspace & 255) != 0 || workspace_bytes < odmkv_quantize_workspace_bytes(chunk->cap)) return ODMKV_ERR_WORKSPACE;
    for (int c = 1; c <= 3; ++c)
        if (chunk->cap[c] % 16 != 0) return ODMKV_ERR_SHAPE;
    if (chunk->T <= 0) return ODMKV_ERR_SHAPE;
    if (dtype < 0 || dtype > 2) return ODMKV_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    QuantArgs a;
    a.K = K; a.V = V; a.bits = bits; a.pi_k = pi_k; a.pi_v = pi_v; a.codebooks = codebooks;
    a.ch = *chunk;
    const int BH = chunk->B * chunk->H;
    a.ntiles = (chunk->T + kTile - 1) / kTile;
    a.tile_base = (const int32_t *)plan_workspace + (size_t)BH * a.ntiles * kNumClasses;
    {
        size_t off = 0;
        for (int li = 0; li < 3; ++li) {
            const size_t bytes = ((size_t)chunk->cap[li + 1] * 16 * qbits(li) + 255) / 256 * 256;
            a.k_scratch[li] = (uint8_t *)workspace + off;
            a.v_scratch[li] = (uint8_t *)workspace + off + bytes;
            off += 2 * bytes;
        }
    }
    long long n_work = (long long)BH * a.ntiles * 4;   // quarter tiles; each is visited by a key group and a value group
    int grid = 2 * (int)((n_work + 1) / 2 < num_sms() / 2 ? (n_work + 1) / 2 : num_sms() / 2);
    dim3 pad_grid(BH, kNumClasses);
    cudaError_t e;
#define ODMKV_LAUNCH_Q(DT)                                                                                   \
    e = cudaFuncSetAttribute(quantize_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kQuantKernelSmem); \
    if (e != cudaSuccess) return (int)e;                                                                     \
    e = cudaFuncSetAttribute(quantize_kernel<DT>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared); \
    if (e != cudaSuccess) return (int)e;                                                                     \
    fill_padding_kernel<DT><<<pad_grid, 128, 0, st>>>(*chunk, a.k_scratch[0], a.k_scratch[1], a.k_scratch[2], a.v_scratch[0], a.v_scratch[1], a.v_scratch[2]);  \
    timing_begin("quantize", st);                                                                            \
    quantize_kernel<DT><<<grid, 512, kQuantKernelSmem, st>>>(a);                                                   \
    timing_end(st);
    // 16-bit caches take the tcgen05 kernel (whole plan tiles, two CTAs per SM, even CTAs keys / odd CTAs values)
    const long long n_tiles_side = (long long)BH * a.ntiles;
    const int grid_u = 2 * (int)(n_tiles_side < num_sms() ? n_tiles_side : num_sms());
    unsigned *qstatus = quant_status_ptr();
#define ODMKV_LAUNCH_QU(DT)                                                                                  \
    if (!qstatus) return ODMKV_ERR_UNSUPPORTED;                                                              \
    e = cudaFuncSetAttribute(quantize_umma_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)umma::kSmemBytes); \
    if (e != cudaSuccess) return (int)e;                                                                     \
    fill_padding_kernel<DT><<<pad_grid, 128, 0, st>>>(*chunk, a.k_scratch[0], a.k_scratch[1], a.k_scratch[2], a.v_scratch[0], a.v_scratch[1], a.v_scratch[2]);  \
    timing_begin("quantize", st);                                                                            \
    quantize_umma_kernel<DT><<<grid_u, umma::kThreads, umma::kSmemBytes, st>>>(a, qstatus);                    \
    timing_end(st);
    if (dtype == kF16) { ODMKV_LAUNCH_QU(kF16) } else if (dtype == kBF16) { ODMKV_LAUNCH_QU(kBF16) } else { ODMKV_LAUNCH_Q(kF32) }
#undef ODMKV_LAUNCH_QU
#undef ODMKV_LAUNCH_Q
    // 2/3/4-bit banks: linear scratch -> tile layout
    for (int li = 0; li < 3; ++li) {
        const int ntile = chunk->cap[li + 1] / 16;
        if (ntile <= 0) continue;
        int rg = (ntile + 7) / 8;
        if (rg > 16 * num_sms()) rg = 16 * num_sms();
        if (li == 0) {
            retile_kernel<2, true><<<rg, 256, 0, st>>>(a.k_scratch[0], chunk->k_codes[0], ntile);
            retile_kernel<2, false><<<rg, 256, 0, st>>>(a.v_scratch[0], chunk->v_codes[0], ntile);
        } else if (li == 1) {
            retile_kernel<3, true><<<rg, 256, 0, st>>>(a.k_scratch[1], chunk->k_codes[1], ntile);
            retile_kernel<3, false><<<rg, 256, 0, st>>>(a.v_scratch[1], chunk->v_codes[1], ntile);
        } else {
            retile_kernel<4, true><<<rg, 256, 0, st>>>(a.k_scratch[2], chunk->k_codes[2], ntile);
            retile_kernel<4, false><<<rg, 256, 0, st>>>(a.v_scratch[2], chunk->v_codes[2], ntile);
        }
    }
    return launch_status();
}

int odmkv_compact_chunks(const odmkv_chunk *src, int n_src, const odmkv_chunk *dst, const int32_t *dst_off, int dtype,
                         void *workspace, size_t workspace_bytes, void *stream) {
    if (!src || !dst || !dst_off || !workspace) return ODMKV_ERR_ARG;
    if (n_src <= 0 || n_src > kMaxChunks) return ODMKV_ERR_LIMIT;
    int rc = check_chunk(dst);
    if (rc) return rc;
    for (int i = 0; i < n_src; ++i) {
        rc = check_chunk(&src[i]);
        if (rc) return rc;
        if (src[i].B != dst->B || src[i].H != dst->H) return ODMKV_ERR_SHAPE;
    }
    if (dtype < 0 || dtype > 2) return ODMKV_ERR_UNSUPPORTED;
    if (((uintptr_t)workspace & 255) != 0 || workspace_bytes < odmkv_quantize_workspace_bytes(dst->cap)) return ODMKV_ERR_WORKSPACE;
    for (int c = 1; c <= 3; ++c)
        if (dst->cap[c] % 16 != 0) return ODMKV_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    CompactArgs a;
    for (int i = 0; i < n_src; ++i) a.src[i] = src[i];
    a.dst = *dst; a.dst_off = dst_off; a.n_src = n_src;
    size_t off = 0;
    for (int li = 0; li < 3; ++li) {
        const size_t bytes = ((size_t)dst->cap[li + 1] * 16 * qbits(li) + 255) / 256 * 256;
        a.k_scratch[li] = (uint8_t *)workspace + off;
        a.v_scratch[li] = (uint8_t *)workspace + off + bytes;
        off += 2 * bytes;
    }
    cudaMemsetAsync(workspace, 0, off, st);   // padding slots of the linear rows: zero codes
    dim3 grid(dst->B * dst->H, n_src, kNumClasses);
    if (dtype == kF16) compact_gather_kernel<kF16><<<grid, 256, 0, st>>>(a);
    else if (dtype == kBF16) compact_gather_kernel<kBF16><<<grid, 256, 0, st>>>(a);
    else compact_gather_kernel<kF32><<<grid, 256, 0, st>>>(a);
    for (int li = 0; li < 3; ++li) {
        const int ntile = dst->cap[li + 1] / 16;
        if (ntile <= 0) continue;
        int rg = (ntile + 7) / 8;
        if (rg > 16 * num_sms()) rg = 16 * num_sms();
        if (li == 0) {
            retile_kernel<2, true><<<rg, 256, 0, st>>>(a.k_scratch[0], dst->k_codes[0], ntile);
            retile_kernel<2, false><<<rg, 256, 0, st>>>(a.v_scratch[0], dst->v_codes[0], ntile);
        } else if (li == 1) {
            retile_kernel<3, true><<<rg, 256, 0, st>>>(a.k_scratch[1], dst->k_codes[1], ntile);
            retile_kernel<3, false><<<rg, 256, 0, st>>>(a.v_scratch[1], dst->v_codes[1], ntile);
        } else {
            retile_kernel<4, true><<<rg, 256, 0, st>>>(a.k_scratch[2], dst->k_codes[2], ntile);
            retile_kernel<4, false><<<rg, 256, 0, st>>>(a.v_scratch[2], dst->v_codes[2], ntile);
        }
    }
    return launch_status();
}

int odmkv_encode_pack(const float *y, long long n, int bits, const float *codebook, uint8_t *out, void *stream) {
    if (!y || !codebook || !out) return ODMKV_ERR_ARG;
    int c = class_of_bits(bits);
    if (c < 1 || c > 4) return ODMKV_ERR_UNSUPPORTED;
    if (n <= 0) return n == 0 ? ODMKV_OK : ODMKV_ERR_SHAPE;
    long long blocks = (n + 7) / 8;
    int grid = (int)(blocks < 4 * num_sms() ? blocks : 4 * num_sms());
    encode_pack_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(y, n, c - 1, codebook, out);
    return launch_status();
}

int odmkv_dequant_chunk(const odmkv_chunk *chunk, int in_dtype, const float *pi_k, const float *pi_v,
                        const float *codebooks, void *K_out, void *V_out, int out_dtype, int T_dense,
                        int include_exact, void *stream) {
    if (!pi_k || !pi_v || !codebooks || !K_out || !V_out) return ODMKV_ERR_ARG;
    int rc = check_chunk(chunk);
    if (rc) return rc;
    if (in_dtype < 0 || in_dtype > 2 || out_dtype < 0 || out_dtype > 2) return ODMKV_ERR_UNSUPPORTED;
    if (T_dense <= 0) return ODMKV_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    DequantArgs a;
    a.ch = *chunk; a.pi_k = pi_k; a.pi_v = pi_v; a.codebooks = codebooks; a.K_out = K_out; a.V_out = V_out; a.T_dense = T_dense;
    a.tiles_before[0] = 0;
    for (int li = 0; li < 4; ++li) a.tiles_before[li + 1] = a.tiles_before[li] + (chunk->cap[li + 1] + kTile - 1) / kTile;
    cudaError_t e;
    if (a.tiles_before[4] > 0) {
        int grid = a.tiles_before[4] < num_sms() ? a.tiles_before[4] : num_sms();
#define ODMKV_LAUNCH_D(ODT)                                                                                      \
    e = cudaFuncSetAttribute(dequant_kernel<ODT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDequantSmem); \
    if (e != cudaSuccess) return (int)e;                                                                         \
    dequant_kernel<ODT><<<grid, 256, kDequantSmem, st>>>(a);
        if (out_dtype == kF16) { ODMKV_LAUNCH_D(kF16) } else if (out_dtype == kBF16) { ODMKV_LAUNCH_D(kBF16) } else { ODMKV_LAUNCH_D(kF32) }
#undef ODMKV_LAUNCH_D
    }
    if (include_exact && chunk->cap[5] > 0) {
        int grid = (chunk->cap[5] + 7) / 8;
        if (grid > 8 * num_sms()) grid = 8 * num_sms();
#define ODMKV_LAUNCH_E(IDT, ODT) scatter_exact_kernel<IDT, ODT><<<grid, 256, 0, st>>>(*chunk, K_out, V_out, T_dense);
        if (in_dtype == kF16) {
            if (out_dtype == kF16) { ODMKV_LAUNCH_E(kF16, kF16) } else if (out_dtype == kBF16) { ODMKV_LAUNCH_E(kF16, kBF16) } else { ODMKV_LAUNCH_E(kF16, kF32) }
        } else if (in_dtype == kBF16) {
            if (out_dtype == kF16) { ODMKV_LAUNCH_E(kBF16, kF16) } else if (out_dtype == kBF16) { ODMKV_LAUNCH_E(kBF16, kBF16) } else { ODMKV_LAUNCH_E(kBF16, kF32) }
        } else {
            if (out_dtype == kF16) { ODMKV_LAUNCH_E(kF32, kF16) } else if (out_dtype == kBF16) { ODMKV_LAUNCH_E(kF32, kBF16) } else { ODMKV_LAUNCH_E(kF32, kF32) }
        }
#undef ODMKV_LAUNCH_E
    }
    return launch_status();
}

int odmkv_export_bank(const odmkv_chunk *chunk, int class_idx, const int32_t *row_start, uint8_t *indices_k,
                      uint8_t *indices_v, float *norms_k, float *norms_v, int64_t *positions, void *stream) {
    int rc = check_chunk(chunk);
    if (rc) return rc;
    if (class_idx < 1 || class_idx > 4) return ODMKV_ERR_ARG;
    if (!row_start || !indices_k || !indices_v || !norms_k || !norms_v || !positions) return ODMKV_ERR_ARG;
    export_bank_kernel<<<chunk->B * chunk->H, 256, 0, (cudaStream_t)stream>>>(*chunk, class_idx, row_start, indices_k, indices_v,
                                                                            norms_k, norms_v, positions);
    return launch_status();
}

int odmkv_export_positions(const odmkv_chunk *chunk, int class_idx, const int32_t *row_start, int64_t *positions,
                           void *stream) {
    int rc = check_chunk(chunk);
    if (rc) return rc;
    if ((class_idx != 0 && class_idx != 5) || !row_start || !positions) return ODMKV_ERR_ARG;
    export_positions_kernel<<<chunk->B * chunk->H, 256, 0, (cudaStream_t)stream>>>(*chunk, class_idx, row_start, positions);
    return launch_status();
}

}  // extern "C"
