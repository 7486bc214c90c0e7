// Shared device/host helpers for the odmkv_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/odmkv_b200.h"

namespace odmkv {

constexpr int kD = ODMKV_HEAD_DIM;          // head dimension
constexpr int kTile = ODMKV_TILE;           // tokens per quantise tile
constexpr int kNumClasses = ODMKV_NUM_CLASSES;
constexpr int kSegAlign = ODMKV_SEG_ALIGN;
constexpr int kMaxChunks = 12;              // chunk descriptors that fit in kernel parameters

enum DType : int { kF16 = 0, kBF16 = 1, kF32 = 2 };

// class index: 0 evicted, 1..4 = 2/3/4/8-bit banks, 5 = exact 16-bit bank
__host__ __device__ inline int class_of_bits(int b) {
    switch (b) {
        case 0: return 0;
        case 2: return 1;
        case 3: return 2;
        case 4: return 3;
        case 8: return 4;
        case 16: return 5;
        default: return -1;
    }
}
__host__ __device__ inline int bits_of_qlevel(int li) { return li == 0 ? 2 : li == 1 ? 3 : li == 2 ? 4 : 8; }
// bytes of one packed 128-coordinate code vector for quantised level index li (0..3)
__host__ __device__ inline int code_bytes(int li) { return li == 0 ? 32 : li == 1 ? 48 : li == 2 ? 64 : 128; }
// bytes per row in the reference's bank layout (3-bit codes are stored as nibbles there)
__host__ __device__ inline int ref_code_bytes(int li) { return li == 0 ? 32 : li == 3 ? 128 : 64; }
__host__ __device__ inline int dtype_size(int dt) { return dt == kF32 ? 4 : 2; }

// optional event timing of the dominant kernels (timing.cu)
bool timing_on();
void timing_begin(const char *name, cudaStream_t st);
void timing_end(cudaStream_t st);

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ODMKV_OK : (int)e;
}

// ---- element loads / stores in the cache dtype -------------------------------------------------
template <int DT> struct Elem;
template <> struct Elem<kF16> {
    using T = __half;
    __device__ static float to_f32(T v) { return __half2float(v); }
    __device__ static T from_f32(float v) { return __float2half_rn(v); }
};
template <> struct Elem<kBF16> {
    using T = __nv_bfloat16;
    __device__ static float to_f32(T v) { return __bfloat162float(v); }
    __device__ static T from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<kF32> {
    using T = float;
    __device__ static float to_f32(T v) { return v; }
    __device__ static T from_f32(float v) { return v; }
};

// load 4 consecutive elements starting at element index e (e % 4 == 0) as fp32
template <int DT>
__device__ inline float4 load4(const void *base, size_t e) {
    if constexpr (DT == kF32) {
        return *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(base) + e);
    } else if constexpr (DT == kF16) {
        uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(base) + e);
        float2 a = __half22float2(*reinterpret_cast<__half2 *>(&raw.x));
        float2 b = __half22float2(*reinterpret_cast<__half2 *>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    } else {
        uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __nv_bfloat16 *>(base) + e);
        float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&raw.x));
        float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
}

template <int DT>
__device__ inline void store4(void *base, size_t e, float4 v) {
    if constexpr (DT == kF32) {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(base) + e) = v;
    } else if constexpr (DT == kF16) {
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t *>(&a);
        raw.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(base) + e) = raw;
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t *>(&a);
        raw.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(base) + e) = raw;
    }
}

// ---- nearest centroid: searchsorted(left) then the nearer neighbour, lower index on ties --------
__device__ inline int nearest_centroid(float y, const float *c, int k) {
    int lo = 0, hi = k;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (c[mid] < y) lo = mid + 1; else hi = mid;
    }
    int a = lo - 1 < 0 ? 0 : lo - 1;
    int b = lo > k - 1 ? k - 1 : lo;
    float da = fabsf(__fsub_rn(y, c[a]));
    float db = fabsf(__fsub_rn(y, c[b]));
    return (da <= db) ? a : b;
}

// ---- bank layouts ---------------------------------------------------------------------------------
// 8-bit bank (li = 3): token-major, 128 bytes per slot, byte d = code of coordinate d (keys and values).
//
// 2/3/4-bit banks (li = 0..2, b bits per code): slots are grouped in tiles of 16 (256*b bytes per tile).
// A tile is laid out for the m16n8k16 tensor-core fragments of the decode kernel: lane (g, t) of a warp
// (g = lane / 4, t = lane % 4) owns the 8*b bytes at tile + lane * 8 * b, as 32 "pair fields" of 2*b bits
// (low code in the low bits), packed little-endian in ascending field order.
//   keys:   field 4 s + 2 odd + hi holds coordinates (32 t + 4 s + 2 odd, + 1) of slot g + 8 hi, i.e. the
//           four fields of step s are the A registers a0..a3 of that HMMA step, in order;
//   values: field 4 m + 2 hi + a holds coordinate 16 m + g + 8 a of tokens (2 t + 8 hi, 2 t + 8 hi + 1),
//           again a0..a3 of step m.
// The "linear" layout (scratch and odmkv_encode_pack output) is the plain little-endian bit stream of the
// 128 codes of one slot, 16*b bytes per slot.
__host__ __device__ inline int qbits(int li) { return li == 0 ? 2 : li == 1 ? 3 : li == 2 ? 4 : 8; }

__device__ inline uint32_t read_bits(const uint8_t *p, int bitoff, int nbits) {
    const int byte = bitoff >> 3, sh = bitoff & 7;
    uint32_t v = (uint32_t)p[byte] >> sh;
    if (sh + nbits > 8) v |= (uint32_t)p[byte + 1] << (8 - sh);
    return v & ((1u << nbits) - 1u);
}

__device__ inline int k_code(const uint8_t *bank, int li, long long slot, int d) {
    if (li == 3) return bank[(size_t)slot * 128 + d];
    const int b = qbits(li);
    const long long tile = slot >> 4;
    const int r = (int)(slot & 15), g = r & 7, hi = r >> 3, t = d >> 5, f = (d & 31) >> 1;
    const int field = 4 * (f >> 1) + 2 * (f & 1) + hi;
    return (int)read_bits(bank + (size_t)tile * 256 * b + (size_t)(g * 4 + t) * 8 * b, field * 2 * b + (d & 1) * b, b);
}

__device__ inline int v_code(const uint8_t *bank, int li, long long slot, int d) {
    if (li == 3) return bank[(size_t)slot * 128 + d];
    const int b = qbits(li);
    const long long tile = slot >> 4;
    const int r = (int)(slot & 15), m = d >> 4, dd = d & 15, g = dd & 7, a = dd >> 3;
    const int t = (r & 7) >> 1, e = r & 1, hi = r >> 3;
    return (int)read_bits(bank + (size_t)tile * 256 * b + (size_t)(g * 4 + t) * 8 * b, (4 * m + hi * 2 + a) * 2 * b + e * b, b);
}

__device__ inline int linear_code(const uint8_t *rows, int li, long long slot, int d) {
    const int b = qbits(li);
    return (int)read_bits(rows + (size_t)slot * 16 * b, d * b, b);
}

__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace odmkv
