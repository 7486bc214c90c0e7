// Decode attention over packed chunks (sm_100a) -- split-K flash decoding in code space.
//
// Replaces the q_len = 1 attention call behind the reference's wrapper
// (kvquant/attention_patch.py:30-55) and the dense dequantised cache it reads
// (kvquant/tq_adaptive_backend.py:205-242).  Identity used: with q' = pi_k q,
//   q . k_hat_j = norm^K_j * sum_i q'_i c[idxK_{j,i}],
//   out = (sum_j p_j norm^V_j c[idxV_j]) pi_v  +  sum_{j exact} p_j v_j,
// so every quantised token is consumed as codes + two norms; rotation is applied once to the
// queries (prologue kernel) and once to the merged accumulator (merge kernel).  Evicted tokens are
// in no bank and therefore absent, which is what the reference's fake-key mask achieves.
//
// Grid: (n_splits, B*H).  Each CTA takes the same fraction of every (chunk, class) segment of its
// (b, h), keeps per-warp running (max, sum, accumulators) for the G query heads of the KV head and
// writes one partial; the merge kernel combines partials with a log-sum-exp merge.
#include "decode_shared.cuh"

namespace odmkv {

constexpr int kDecThreads = 128;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kMaxSlots = 160;   // partial slots per (b, h) the merge kernel accepts

// rotate the queries once: qrot[r][i] = sum_j pi_k[i][j] q[r][j]; also keep q as fp32.
// Warp w owns output rows w, w+4, ..., w+124: every lane loads its four columns of all 32 rows
// (32 independent, coalesced 16-byte loads), then a reduce-scatter leaves row (w + 4*lane) in lane `lane`.
template <int QDT>
__global__ void __launch_bounds__(kD) rotate_q_kernel(const void *__restrict__ q, const float *__restrict__ pi_k, float *__restrict__ qrot,
                                                       float *__restrict__ qf) {
    __shared__ __align__(16) float qs[kD];
    const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    qs[tid] = Elem<QDT>::to_f32(reinterpret_cast<const typename Elem<QDT>::T *>(q)[(size_t)r * kD + tid]);
    __syncthreads();
    qf[(size_t)r * kD + tid] = qs[tid];
    const float4 qv = *reinterpret_cast<const float4 *>(qs + 4 * lane);
    float v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const float4 p = *reinterpret_cast<const float4 *>(pi_k + (size_t)(warp + 4 * k) * kD + 4 * lane);
        float acc = p.x * qv.x;
        acc = fmaf(p.y, qv.y, acc);
        acc = fmaf(p.z, qv.z, acc);
        v[k] = fmaf(p.w, qv.w, acc);
    }
#pragma unroll
    for (int o = 16, n = 16; o >= 1; o >>= 1, n >>= 1) {
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int k = 0; k < n; ++k) {
            const float send = upper ? v[k] : v[k + n];
            const float keep = upper ? v[k + n] : v[k];
            v[k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
    }
    qrot[(size_t)r * kD + warp + 4 * lane] = v[0];
}

// per-warp online-softmax state for GP query heads; each lane owns coordinates 4*lane .. 4*lane+3
template <int GP>
struct WarpState {
    float m[GP], l[GP];
    float ar[GP][4];  // code-space accumulator (to be rotated by pi_v)
    float ae[GP][4];  // exact-space accumulator
};

// fold the logits of up to 32 tokens (one per lane) into the running state; returns p per head
template <int GP>
__device__ inline void softmax_step(WarpState<GP> &st, const float (&logit)[GP], bool valid, float (&p)[GP]) {
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        float x = valid ? logit[g] : -INFINITY;
        float mx = warp_max(x);
        float mn = fmaxf(st.m[g], mx);
        float corr = (st.m[g] == -INFINITY) ? 0.f : __expf(st.m[g] - mn);
        float pv = (valid && mn > -INFINITY) ? __expf(x - mn) : 0.f;
        st.l[g] = st.l[g] * corr + warp_sum(pv);
        st.m[g] = mn;
#pragma unroll
        for (int d = 0; d < 4; ++d) { st.ar[g][d] *= corr; st.ae[g][d] *= corr; }
        p[g] = pv;
    }
}

// one group of up to 32 slots of a quantised bank; lane = token for the key dot products, lane = four
// coordinates for the value accumulation.  Codes are read through the layout accessors, so this path
// serves every level (it is the plain, slow reader; the tensor-core kernel is the fast one).
template <int GP>
__device__ inline void process_codes(WarpState<GP> &st, const odmkv_chunk &ch, int li, int s_begin, int s_end,
                                     const float *__restrict__ lut, const float *__restrict__ qs, float scale, int lane) {
    const int s = s_begin + lane;
    const bool valid = s < s_end;
    float logit[GP], p[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) logit[g] = 0.f;
    if (valid) {
        const uint8_t *bank = ch.k_codes[li];
        for (int i = 0; i < kD; ++i) {
            const float c = lut[k_code(bank, li, s, i)];
#pragma unroll
            for (int g4 = 0; g4 < GP / 4; ++g4) {
                float4 qv = *reinterpret_cast<const float4 *>(qs + i * GP + 4 * g4);
                logit[4 * g4] = fmaf(c, qv.x, logit[4 * g4]);
                logit[4 * g4 + 1] = fmaf(c, qv.y, logit[4 * g4 + 1]);
                logit[4 * g4 + 2] = fmaf(c, qv.z, logit[4 * g4 + 2]);
                logit[4 * g4 + 3] = fmaf(c, qv.w, logit[4 * g4 + 3]);
            }
        }
        const float kn = ch.k_norm[li][s] * scale;
#pragma unroll
        for (int g = 0; g < GP; ++g) logit[g] *= kn;
    }
    softmax_step<GP>(st, logit, valid, p);
    if (valid) {
        const float vn = ch.v_norm[li][s];
#pragma unroll
        for (int g = 0; g < GP; ++g) p[g] *= vn;
    }
    const int cnt = min(32, s_end - s_begin);
    const uint8_t *vbank = ch.v_codes[li];
    for (int j = 0; j < cnt; ++j) {
        float c[4];
#pragma unroll
        for (int d = 0; d < 4; ++d) c[d] = lut[v_code(vbank, li, s_begin + j, 4 * lane + d)];
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            float pj = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
            for (int d = 0; d < 4; ++d) st.ar[g][d] = fmaf(pj, c[d], st.ar[g][d]);
        }
    }
}

// one group of up to 32 exact rows (cache dtype, not rotated); rows [r_begin, r_end) of a dense array
template <int CDT, int GP>
__device__ inline void process_exact(WarpState<GP> &st, const void *__restrict__ kbase, const void *__restrict__ vbase, size_t r_begin,
                                     size_t r_end, const float *__restrict__ qx, float scale, int lane) {
    const size_t r = r_begin + lane;
    const bool valid = r < r_end;
    float logit[GP], p[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) logit[g] = 0.f;
    if (valid) {
        // eight independent loads in flight per step (a lane walks its own row, so nothing here is coalesced and the
        // loop is bound by load latency unless the loads are issued in batches)
        for (int i0 = 0; i0 < kD / 4; i0 += 8) {
            float4 kv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) kv[u] = load4<CDT>(kbase, r * kD + 4 * (i0 + u));
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float kk[4] = {kv[u].x, kv[u].y, kv[u].z, kv[u].w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int g = 0; g < GP; ++g) logit[g] = fmaf(kk[e], qx[(4 * (i0 + u) + e) * GP + g], logit[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < GP; ++g) logit[g] *= scale;
    }
    softmax_step<GP>(st, logit, valid, p);
    const int cnt = (int)min((size_t)32, r_end - r_begin);
    for (int j0 = 0; j0 < cnt; j0 += 8) {     // value rows in batches of eight loads as well (cnt is warp-uniform)
        float4 vv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            vv[u] = j0 + u < cnt ? load4<CDT>(vbase, (r_begin + j0 + u) * kD + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (j0 + u >= cnt) break;
            const float c[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
            for (int g = 0; g < GP; ++g) {
                float pj = __shfl_sync(0xffffffffu, p[g], j0 + u);
#pragma unroll
                for (int d = 0; d < 4; ++d) st.ae[g][d] = fmaf(pj, c[d], st.ae[g][d]);
            }
        }
    }
}

template <int CDT, int GP>
__global__ void __launch_bounds__(kDecThreads) decode_main_kernel(const DecodeChunks chunks, const DecodeArgs a) {
    __shared__ __align__(16) float qs[kD * GP];   // rotated queries, [i][g]
    __shared__ __align__(16) float qx[kD * GP];   // plain queries, [i][g]
    __shared__ float lut[4 * 256];
    __shared__ float red_acc[kDecWarps][GP][2][kD];
    __shared__ float red_m[kDecWarps][GP], red_l[kDecWarps][GP];

    const int bh = blockIdx.y, split = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int BH = a.B * a.H, G = a.G;
    for (int e = tid; e < kD * GP; e += kDecThreads) {
        int i = e / GP, g = e % GP;
        const size_t qi = ((size_t)bh * G + g) * kD + i;
        if (a.q_raw) {   // exact rows and tail only: the plain queries straight from the caller's tensor
            float v = 0.f;
            if (g < G) {
                if (a.q_dtype == kF16) v = __half2float(reinterpret_cast<const __half *>(a.q_raw)[qi]);
                else if (a.q_dtype == kBF16) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(a.q_raw)[qi]);
                else v = reinterpret_cast<const float *>(a.q_raw)[qi];
            }
            qs[e] = 0.f;
            qx[e] = v;
        } else {
            qs[e] = g < G ? a.qrot[qi] : 0.f;
            qx[e] = g < G ? a.qf[qi] : 0.f;
        }
    }
    for (int e = tid; e < 4 * 256; e += kDecThreads) lut[e] = a.codebooks[e];
    __syncthreads();

    WarpState<GP> st;
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        st.m[g] = -INFINITY; st.l[g] = 0.f;
#pragma unroll
        for (int d = 0; d < 4; ++d) { st.ar[g][d] = 0.f; st.ae[g][d] = 0.f; }
    }

    for (int ci = 0; ci < chunks.n; ++ci) {
        const odmkv_chunk &ch = chunks.ch[ci];
        for (int c = 1; c <= 5; ++c) {
            if (!((a.class_mask >> c) & 1)) continue;
            const int cnt = ch.seg_count[c * BH + bh];
            if (cnt == 0) continue;
            const int s0 = ch.seg_start[c * BH + bh];
            const int ngroups = (cnt + 31) / 32;
            const int g_lo = (int)((long long)ngroups * split / a.nsplit), g_hi = (int)((long long)ngroups * (split + 1) / a.nsplit);
            for (int gi = g_lo + warp; gi < g_hi; gi += kDecWarps) {
                const int sb = s0 + gi * 32, se = min(s0 + cnt, sb + 32);
                if (c <= 4) process_codes<GP>(st, ch, c - 1, sb, se, lut + (c - 1) * 256, qs, a.scale, lane);
                else process_exact<CDT, GP>(st, ch.exact_k, ch.exact_v, (size_t)sb, (size_t)se, qx, a.scale, lane);
            }
        }
    }
    // the tail length is a launch argument, or lives in device memory when the launch is replayed from a graph
    // while the tail grows
    const int tail_len = a.tail_len_dev ? max(0, min(__ldg(a.tail_len_dev) + a.tail_len_add, a.tail_cap)) : a.tail_len;
    if (tail_len > 0 && ((a.class_mask >> 6) & 1)) {
        const int ngroups = (tail_len + 31) / 32;
        const int g_lo = (int)((long long)ngroups * split / a.nsplit), g_hi = (int)((long long)ngroups * (split + 1) / a.nsplit);
        const size_t base = (size_t)bh * a.tail_cap;
        for (int gi = g_lo + warp; gi < g_hi; gi += kDecWarps) {
            const size_t rb = base + (size_t)gi * 32, re = min(base + (size_t)tail_len, rb + 32);
            process_exact<CDT, GP>(st, a.tail_k, a.tail_v, rb, re, qx, a.scale, lane);
        }
    }

    // ---- combine the warps of this CTA
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        if (lane == 0) { red_m[warp][g] = st.m[g]; red_l[warp][g] = st.l[g]; }
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            red_acc[warp][g][0][4 * lane + d] = st.ar[g][d];
            red_acc[warp][g][1][4 * lane + d] = st.ae[g][d];
        }
    }
    __syncthreads();
    for (int e = tid; e < GP * 2 * kD; e += kDecThreads) {
        const int g = e / (2 * kD), rest = e % (2 * kD);
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, red_m[w][g]);
        float v = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            float f = red_m[w][g] == -INFINITY ? 0.f : __expf(red_m[w][g] - mm);
            v += (&red_acc[w][g][0][0])[rest] * f;
            l += red_l[w][g] * f;
        }
        const size_t pi = ((size_t)bh * a.nslots + a.slot_base + split) * GP + g;
        a.part_acc[pi * 2 * kD + rest] = v;
        if (rest == 0) { a.part_ml[pi * 2] = mm; a.part_ml[pi * 2 + 1] = l; }
    }
}

// merge the split partials of one query head, rotate the code-space part by pi_v, normalise
template <int ODT>
__global__ void __launch_bounds__(kD) decode_merge_kernel(const float *__restrict__ part_ml, const float *__restrict__ part_acc,
                                                           const float *__restrict__ pi_v, int G, int GP, int nsplit,
                                                           void *__restrict__ out, float *__restrict__ lse, int n_main, int n_cta, int BH) {
    __shared__ float ar[kD];
    __shared__ float w[kMaxSlots];
    __shared__ float sh_ml[2];
    const int r = blockIdx.x;          // bh * G + g
    const int bh = r / G, g = r % G, j = threadIdx.x;
    // Slots in use: all of them, or (n_cta > 0) the first `cnt` main slots -- one per CTA of the persistent
    // tensor-core kernel that overlaps this unit -- followed by the slots from n_main on.
    int cnt = nsplit, skip = 0;
    if (n_cta > 0) {
        const int first = (int)(((long long)bh * n_cta) / BH);
        const int last = (int)((((long long)bh + 1) * n_cta + BH - 1) / BH) - 1;
        cnt = last - first + 1;
        skip = n_main - cnt;
    }
    const int n_used = nsplit - skip;
    if (j < 32) {
        float m = -INFINITY;
        for (int u = j; u < n_used; u += 32) {
            const int s = u < cnt ? u : u + skip;
            m = fmaxf(m, part_ml[(((size_t)bh * nsplit + s) * GP + g) * 2]);
        }
        m = warp_max(m);
        float l = 0.f;
        for (int u = j; u < n_used; u += 32) {
            const int s = u < cnt ? u : u + skip;
            const float *p = part_ml + (((size_t)bh * nsplit + s) * GP + g) * 2;
            float f = p[0] == -INFINITY ? 0.f : __expf(p[0] - m);
            w[u] = f;
            l += p[1] * f;
        }
        l = warp_sum(l);
        if (j == 0) { sh_ml[0] = m; sh_ml[1] = l; }
    }
    __syncthreads();
    float accr = 0.f, acce = 0.f;
#pragma unroll 16
    for (int u = 0; u < n_used; ++u) {
        const int s = u < cnt ? u : u + skip;
        const float *p = part_acc + (((size_t)bh * nsplit + s) * GP + g) * 2 * kD;
        accr = fmaf(p[j], w[u], accr);
        acce = fmaf(p[kD + j], w[u], acce);
    }
    ar[j] = accr;
    __syncthreads();
    // four interleaved partial sums keep 32 loads of the rotation in flight per thread
    float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i0 = 0; i0 < kD; i0 += 32) {
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) pv[i] = __ldg(pi_v + (size_t)(i0 + i) * kD + j);
#pragma unroll
        for (int i = 0; i < 32; ++i) o4[i & 3] = fmaf(ar[i0 + i], pv[i], o4[i & 3]);
    }
    float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    const float l = sh_ml[1];
    o = l > 0.f ? (o + acce) / l : 0.f;
    reinterpret_cast<typename Elem<ODT>::T *>(out)[(size_t)r * kD + j] = Elem<ODT>::from_f32(o);
    if (lse && j == 0) lse[r] = l > 0.f ? sh_ml[0] + logf(l) : -INFINITY;
}

void launch_rotate_q(const void *q, int q_dtype, const float *pi_k, const DecodeWs &ws, int R, cudaStream_t st) {
    if (q_dtype == kF16) rotate_q_kernel<kF16><<<R, kD, 0, st>>>(q, pi_k, ws.qrot, ws.qf);
    else if (q_dtype == kBF16) rotate_q_kernel<kBF16><<<R, kD, 0, st>>>(q, pi_k, ws.qrot, ws.qf);
    else rotate_q_kernel<kF32><<<R, kD, 0, st>>>(q, pi_k, ws.qrot, ws.qf);
}

void launch_decode_cuda_core(const DecodeChunks &dc, const DecodeArgs &a, int cache_dtype, cudaStream_t st) {
    const int GP = round_gp(a.G);
    dim3 grid(a.nsplit, a.B * a.H);
#define ODMKV_DEC(CDT)                                                                           \
    if (GP == 4) decode_main_kernel<CDT, 4><<<grid, kDecThreads, 0, st>>>(dc, a);                \
    else decode_main_kernel<CDT, 8><<<grid, kDecThreads, 0, st>>>(dc, a);
    if (cache_dtype == kF16) { ODMKV_DEC(kF16) } else if (cache_dtype == kBF16) { ODMKV_DEC(kBF16) } else { ODMKV_DEC(kF32) }
#undef ODMKV_DEC
}

void launch_decode_merge(const DecodeWs &ws, const float *pi_v, int BH, int G, int nslots, void *out, int out_dtype, float *lse,
                         cudaStream_t st, int n_main, int n_cta) {
    const int R = BH * G, GP = round_gp(G);
    if (out_dtype == kF16) decode_merge_kernel<kF16><<<R, kD, 0, st>>>(ws.part_ml, ws.part_acc, pi_v, G, GP, nslots, out, lse, n_main, n_cta, BH);
    else if (out_dtype == kBF16) decode_merge_kernel<kBF16><<<R, kD, 0, st>>>(ws.part_ml, ws.part_acc, pi_v, G, GP, nslots, out, lse, n_main, n_cta, BH);
    else decode_merge_kernel<kF32><<<R, kD, 0, st>>>(ws.part_ml, ws.part_acc, pi_v, G, GP, nslots, out, lse, n_main, n_cta, BH);
}

int decode_check_args(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype, const void *tail_k,
                      const void *tail_v, int tail_len, int tail_cap, const float *pi_k, const float *pi_v, const float *codebooks,
                      int B, int H, int G, void *out, int out_dtype, int n_splits, void *workspace, DecodeChunks *dc) {
    if (!q || !pi_k || !pi_v || !codebooks || !out || !workspace) return ODMKV_ERR_ARG;
    if (n_chunks < 0 || n_chunks > kMaxChunks) return ODMKV_ERR_LIMIT;
    if (n_chunks > 0 && !chunks) return ODMKV_ERR_ARG;
    if (B <= 0 || H <= 0 || G <= 0 || G > 8 || (long long)B * H > 65535) return ODMKV_ERR_SHAPE;
    if (q_dtype < 0 || q_dtype > 2 || out_dtype < 0 || out_dtype > 2 || cache_dtype < 0 || cache_dtype > 2) return ODMKV_ERR_UNSUPPORTED;
    if (tail_len < 0 || tail_len > tail_cap || (tail_len > 0 && (!tail_k || !tail_v))) return ODMKV_ERR_ARG;
    if (n_splits <= 0 || n_splits > 128) return ODMKV_ERR_ARG;
    if (((uintptr_t)workspace & 255) != 0) return ODMKV_ERR_WORKSPACE;
    dc->n = n_chunks;
    for (int i = 0; i < n_chunks; ++i) {
        if (chunks[i].B != B || chunks[i].H != H || !chunks[i].seg_start || !chunks[i].seg_count) return ODMKV_ERR_SHAPE;
        dc->ch[i] = chunks[i];
    }
    return ODMKV_OK;
}

}  // namespace odmkv

using namespace odmkv;

extern "C" {

int odmkv_decode_default_splits(int B, int H, long long max_tokens_per_head) {
    // Partial slots per (sample, KV head) that let the tensor-core kernel run one CTA pair per SM of a
    // 148-SM device: the CTAs that can overlap one unit, plus one.  The plain kernel uses the same number of
    // equal splits (at most 64), shortened for short contexts.
    if (B <= 0 || H <= 0) return 1;
    const long long BH = (long long)B * H;
    long long n = (2 * 148 + BH - 1) / BH + 1;
    const long long by_len = (max_tokens_per_head + 255) / 256 + 1;
    if (n > by_len) n = by_len;
    if (n < 2) n = 2;
    if (n > 128) n = 128;
    return (int)n;
}

// room for n_splits partial slots of the main kernel plus the slots of the exact / tail kernel
size_t odmkv_decode_workspace_bytes(int B, int H, int G, int n_splits) {
    if (B <= 0 || H <= 0 || G <= 0 || n_splits <= 0) return 0;
    return decode_ws_layout(B, H, G, n_splits + 8, nullptr, nullptr) + 256;
}

int odmkv_decode_attn(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                      const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                      const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                      int out_dtype, float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                      void *stream) {
    DecodeChunks dc;
    int rc = decode_check_args(q, q_dtype, chunks, n_chunks, cache_dtype, tail_k, tail_v, tail_len, tail_cap, pi_k, pi_v, codebooks,
                               B, H, G, out, out_dtype, n_splits, workspace, &dc);
    if (rc) return rc;
    if (n_splits > 64) return ODMKV_ERR_ARG;
    DecodeWs ws;
    if (workspace_bytes < decode_ws_layout(B, H, G, n_splits, &ws, (unsigned char *)workspace)) return ODMKV_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int BH = B * H;
    launch_rotate_q(q, q_dtype, pi_k, ws, BH * G, st);
    DecodeArgs a;
    a.qrot = ws.qrot; a.qf = ws.qf; a.tail_k = tail_k; a.tail_v = tail_v; a.codebooks = codebooks;
    a.part_ml = ws.part_ml; a.part_acc = ws.part_acc; a.tail_len = tail_len; a.tail_cap = tail_cap;
    a.tail_len_dev = nullptr; a.tail_len_add = 0; a.q_raw = nullptr; a.q_dtype = 0;
    a.B = B; a.H = H; a.G = G; a.nsplit = n_splits; a.slot_base = 0; a.nslots = n_splits; a.class_mask = 0x7e; a.scale = scale;
    timing_begin("decode_main", st);
    launch_decode_cuda_core(dc, a, cache_dtype, st);
    timing_end(st);
    launch_decode_merge(ws, pi_v, BH, G, n_splits, out, out_dtype, lse, st);
    return launch_status();
}

int odmkv_abi_version(void) { return ODMKV_ABI_VERSION; }

const char *odmkv_status_string(int status) {
    switch (status) {
        case ODMKV_OK: return "ok";
        case ODMKV_ERR_ARG: return "invalid argument (null pointer or inconsistent option)";
        case ODMKV_ERR_SHAPE: return "invalid shape";
        case ODMKV_ERR_WORKSPACE: return "workspace too small or not 256-byte aligned";
        case ODMKV_ERR_UNSUPPORTED: return "unsupported dtype or bit width";
        case ODMKV_ERR_LIMIT: return "size beyond a compiled-in limit";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

}  // extern "C"
