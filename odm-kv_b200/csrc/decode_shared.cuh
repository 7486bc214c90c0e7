// Pieces shared by the two decode-attention launchers (decode.cu, decode_mma.cu).
#pragma once
#include "common.cuh"

namespace odmkv {

struct DecodeChunks {
    odmkv_chunk ch[kMaxChunks];
    int n;
};

// Partials: every CTA of either main kernel writes one slot (bh, slot): running max m (natural-log
// domain), denominator l, and two 128-vectors per query head: the code-space accumulator (to be rotated
// by pi_v) and the exact-space accumulator.
struct DecodeWs {
    float *qrot;      // [B*H*G, 128]  pi_k q
    float *qf;        // [B*H*G, 128]  q as fp32
    float *part_ml;   // [BH, nslots, GP, 2]
    float *part_acc;  // [BH, nslots, GP, 2, 128]
};

struct DecodeArgs {
    const float *qrot;
    const float *qf;
    const void *tail_k;
    const void *tail_v;
    const float *codebooks;
    float *part_ml;
    float *part_acc;
    int tail_len, tail_cap;
    const int32_t *tail_len_dev;   // when set: the tail length is read from device memory (plus tail_len_add), bounded by tail_cap
    int tail_len_add;
    const void *q_raw;             // when set: the caller's queries (dtype q_dtype), read directly instead of qf / qrot --
    int q_dtype;                   // for a launch that must not wait for the rotation kernel (no 8-bit codes in it)
    int B, H, G;
    int nsplit;        // CTAs per (b, h) of this launch
    int slot_base;     // first partial slot this launch writes
    int nslots;        // partial slots per (b, h) in the workspace
    int class_mask;    // bit c set: this launch consumes class c (1..5); bit 6: the dense tail
    float scale;
};

__host__ __device__ inline int round_gp(int G) { return G <= 4 ? 4 : 8; }

inline size_t decode_ws_layout(int B, int H, int G, int nslots, DecodeWs *ws, unsigned char *base) {
    const size_t BH = (size_t)B * H, GP = round_gp(G);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = (off + bytes + 255) / 256 * 256; return o; };
    size_t o_qr = take(BH * G * kD * 4), o_qf = take(BH * G * kD * 4), o_ml = take(BH * nslots * GP * 2 * 4),
           o_acc = take(BH * nslots * GP * 2 * kD * 4);
    if (ws && base) {
        ws->qrot = (float *)(base + o_qr); ws->qf = (float *)(base + o_qf);
        ws->part_ml = (float *)(base + o_ml); ws->part_acc = (float *)(base + o_acc);
    }
    return off;
}

// implemented in decode.cu
void launch_rotate_q(const void *q, int q_dtype, const float *pi_k, const DecodeWs &ws, int R, cudaStream_t st);
void launch_decode_cuda_core(const DecodeChunks &dc, const DecodeArgs &a, int cache_dtype, cudaStream_t st);
// n_cta > 0: the first n_main slots of a unit belong to the persistent tensor-core kernel and only those of
// its CTAs that overlap the unit were written
void launch_decode_merge(const DecodeWs &ws, const float *pi_v, int BH, int G, int nslots, void *out, int out_dtype, float *lse,
                         cudaStream_t st, int n_main = 0, int n_cta = 0);
int decode_check_args(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype, const void *tail_k,
                      const void *tail_v, int tail_len, int tail_cap, const float *pi_k, const float *pi_v, const float *codebooks,
                      int B, int H, int G, void *out, int out_dtype, int n_splits, void *workspace, DecodeChunks *dc);

}  // namespace odmkv
