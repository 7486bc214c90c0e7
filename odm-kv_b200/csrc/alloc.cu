// Per-layer Lagrangian bit allocation on the device (sm_100a).
//
// Replaces optimal_scores_to_bits (kvquant/allocator.py:459-663).  One "problem" is the flattened
// score tensor of one (layer, sample).  The search runs as a fixed schedule of rounds; every round
// is one pass over the scores that accumulates a few integers (level counts, or a 16-bit radix
// histogram during gap closure), followed by a tiny state update:
//   rounds 0..73      assignment passes: widen hi (x10 while avg > target, at most 8 times),
//                     64 bisection halvings in fp64, one final pass that records the choice;
//   closure rounds    per level pair: four radix-select passes that find the k-th smallest
//                     (score, index) key among the tokens at a level, one pass that moves them.
// The arithmetic that decides a token's level is three separately rounded fp32 operations
// (s*eps_k, lambda*b_k, their sum) and a first-minimum argmin, exactly as the reference's
// broadcasted torch expression; the average is fl32(total bits) / fl32(n) with an exact integer
// total.  On one GPU the state update runs in the last block of each pass; with KV heads sharded
// over ranks the caller sums the accumulator over ranks between `eval` and `update`.
#include "common.cuh"

#include <cub/device/device_radix_sort.cuh>
#include <mutex>

namespace odmkv {

constexpr int kMaxL = ODMKV_MAX_LEVELS;
constexpr int kAccHead = 16;                 // counts[8], ties, tie_sel, tie_unsel, spare
constexpr int kHistBins = 1 << 16;
constexpr int kAccLen = kAccHead + kHistBins;
constexpr int kEvalRounds = 74;              // 1 + 8 widenings + 64 halvings + 1 final
constexpr int kAllocThreads = 256;
constexpr int kPerThread = 8;
constexpr int kSortLanes = 8;                // sorts of different problems in flight at once (helper streams)

struct AllocCfg {
    float eps32[kMaxL];
    float bits32[kMaxL];
    int levels[kMaxL];
    int K;
    int sink_bits;
    double target;
    double inv_da[kMaxL * kMaxL];   // 1 / (eps32[i] - eps32[j]) in fp64 (0 where the slopes are equal)
};

// Breakpoints of the lower envelope of the K cost lines  s -> eps32[k] * s + lamb[k]  over s >= 0 (exact real
// arithmetic on the fp32 constants, evaluated in fp64).  Between two breakpoints the level of the envelope
// is also the fp32 argmin of the reference's three-operation cost, as long as s stays outside a relative band
// around each breakpoint: the fp32 costs differ from the lines by at most 2^-23 of their value, two lines that
// cross at tau separate by |eps_i - eps_j| * |s - tau|, so a band of 64 * 2^-23 * cost(tau) / |lamb_j - lamb_i|
// (at least 1e-5) is more than enough.  Scores inside a band, and every score when a level that is not on
// the envelope comes within 1e-4 (relative) of it at a breakpoint, are evaluated with the full cost formula.
struct Envelope {
    float lo[kMaxL], hi[kMaxL];   // band [lo, hi] around breakpoint v (v < nh - 1)
    int level[kMaxL];             // level of the envelope between breakpoints v - 1 and v
    int nh;                       // number of envelope pieces; 0 = use the full formula for every score
};

// (Where two cost lines cross is computed as a product with the precomputed reciprocal of the slope difference, a
// relative change of 2^-52 against the quotient; the bands are eleven orders of magnitude wider.  Every loop over
// levels is unrolled over kMaxL so that the lines stay in registers: this routine sits on the critical path of each
// of the 66 dependent steps of a solve.)
__device__ inline void build_envelope(const AllocCfg &cfg, const float *lamb, Envelope &env) {
    const int K = cfg.K;
    double a[kMaxL], c[kMaxL];
#pragma unroll
    for (int k = 0; k < kMaxL; ++k) { a[k] = (double)cfg.eps32[k]; c[k] = (double)lamb[k]; }
    int cur = 0;
    double a_cur = a[0], c_cur = c[0];
#pragma unroll
    for (int k = 1; k < kMaxL; ++k)
        if (k < K && (c[k] < c_cur || (c[k] == c_cur && a[k] < a_cur))) { cur = k; a_cur = a[k]; c_cur = c[k]; }
    const double h0 = c_cur;                       // the envelope at s = 0
    unsigned on = 0u;
    double tau[kMaxL], fv[kMaxL];                  // breakpoint v and the envelope's value there
#pragma unroll
    for (int v = 0; v < kMaxL; ++v) { tau[v] = 0.0; fv[v] = 0.0; }
    int nh = 0;
    double s_cur = 0.0;
    bool ok = true;
    for (int it = 0; it <= kMaxL; ++it) {
        env.level[nh] = cur;
        on |= 1u << cur;
        int nxt = -1;
        double best = 0.0, a_nxt = 0.0, c_nxt = 0.0;
#pragma unroll
        for (int k = 0; k < kMaxL; ++k) {
            if (k < K && k != cur && a[k] < a_cur) {
                const double sx = (c[k] - c_cur) * cfg.inv_da[cur * kMaxL + k];
                if (!(sx < s_cur) && (nxt < 0 || sx < best || (sx == best && a[k] < a_nxt))) { nxt = k; best = sx; a_nxt = a[k]; c_nxt = c[k]; }
            }
        }
        if (nxt < 0) { ++nh; break; }
        const double f = a_cur * best + c_cur;
        const double dc = fabs(c_nxt - c_cur);
        double band = dc > 0.0 ? 64.0 * 1.1920928955078125e-07 * fabs(f) / dc : 1.0;
        if (band < 1e-5) band = 1e-5;
        if (!(band <= 1e-2) || !(best > 0.0) || !(best < 1e37)) ok = false;
#pragma unroll
        for (int v = 0; v < kMaxL; ++v) if (v == nh) { tau[v] = best; fv[v] = f; }
        env.lo[nh] = (float)(best * (1.0 - band) * (1.0 - 1e-7));
        env.hi[nh] = (float)(best * (1.0 + band) * (1.0 + 1e-7));
        ++nh;
        s_cur = best;
        cur = nxt; a_cur = a_nxt; c_cur = c_nxt;
        if (nh >= kMaxL) { ok = false; break; }
    }
    // levels off the envelope must stay clear of it at every breakpoint (their gap is smallest there or at s = 0)
#pragma unroll
    for (int k = 0; k < kMaxL; ++k) {
        if (k < K && !((on >> k) & 1u)) {
#pragma unroll
            for (int v = 0; v + 1 < kMaxL; ++v) {
                if (v + 1 < nh) {
                    const double h = fv[v];
                    const double h_next = v + 2 < nh ? fv[v + 1] : h;
                    const double gk = a[k] * tau[v] + c[k];
                    if (!(gk - h > 1e-4 * fmax(fabs(h), fabs(h_next)))) ok = false;   // 1e-4 >> 2^-22: holds along the whole piece
                }
            }
            if (!(c[k] - h0 > 1e-4 * fabs(h0)) && !(c[k] > h0 && h0 == 0.0)) ok = false;
        }
    }
    env.nh = ok ? nh : 0;
}

struct AllocProblem {
    double lo, hi, lam, gap, gap_before;
    long long level_counts[kMaxL];
    unsigned long long sel_prefix;
    long long sel_k;
    long long n_move;
    int phase;       // 0 widen, 1 bisect, 2 final pass pending, 3 select, 4 apply, 5 done
    int iter, evals, n_active;
    int dir, step, sel_level, sel_to, sel_pass;
    int moved, ties_lambda, ties_cut;
    unsigned ticket;
    unsigned max_finite_bits;
    int any_nonfinite, any_finite;
    Envelope env;    // envelope of the cost lines at `lam` (counting passes)
    int n_sorted;    // live (non-sink) scores of the problem, i.e. the length of its sorted key array
};

struct AllocWs {
    AllocProblem *prob;          // [P]
    unsigned long long *acc;     // [P][kAccLen]
    uint8_t *chosen;             // [P][n]
    AllocCfg *cfg;               // device copy (for the stepwise entry points)
    unsigned *keys_in, *keys_out;   // [P][n] sanitised scores as ordered keys (sinks = 0xffffffff), unsorted / ascending
    void *sort_temp;             // scratch of the radix sort, kSortLanes slices of sort_temp_bytes
    size_t sort_temp_bytes;
    // host-side header kept at the start of the workspace is mirrored in AllocHeader
};

struct AllocHeader {  // lives at the start of the workspace on the device; the host keeps its own copy
    const float *scores;
    const uint8_t *sink_mask;
    int P, n;
    long long idx_base;
};

inline size_t alloc_ws_layout(int P, int n, AllocWs *ws, unsigned char *base) {
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = (off + bytes + 255) / 256 * 256; return o; };
    size_t o_hdr = take(sizeof(AllocHeader)), o_cfg = take(sizeof(AllocCfg)), o_prob = take(sizeof(AllocProblem) * (size_t)P);
    size_t o_acc = take(sizeof(unsigned long long) * (size_t)P * kAccLen), o_ch = take((size_t)P * n);
    size_t sort_bytes = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, sort_bytes, (const unsigned *)nullptr, (unsigned *)nullptr, n);
    sort_bytes = (sort_bytes + 255) / 256 * 256;
    size_t o_ki = take((size_t)P * n * 4), o_ko = take((size_t)P * n * 4), o_st = take(sort_bytes * kSortLanes);
    (void)o_hdr;
    if (ws && base) {
        ws->keys_in = (unsigned *)(base + o_ki); ws->keys_out = (unsigned *)(base + o_ko);
        ws->sort_temp = base + o_st; ws->sort_temp_bytes = sort_bytes;
        ws->cfg = (AllocCfg *)(base + o_cfg);
        ws->prob = (AllocProblem *)(base + o_prob);
        ws->acc = (unsigned long long *)(base + o_acc);
        ws->chosen = (uint8_t *)(base + o_ch);
    }
    return off;
}

// clamp(min=0); when some scores are finite every non-finite one (nan or +inf) becomes the largest
// finite score; when none is finite, nan -> 0 and +inf -> FLT_MAX  (kvquant/allocator.py:543-547)
__device__ inline float sanitize(float s, const AllocProblem &pr) {
    if (s != s) return pr.any_finite ? __uint_as_float(pr.max_finite_bits) : 0.0f;
    s = fmaxf(s, 0.0f);
    if (isinf(s)) s = pr.any_finite ? __uint_as_float(pr.max_finite_bits) : 3.402823466e+38f;
    return s;
}

__device__ inline void refresh_envelope(AllocProblem &pr, const AllocCfg &cfg) {
    const float lam32 = (float)pr.lam;
    float lamb[kMaxL];
    for (int k = 0; k < kMaxL; ++k) lamb[k] = k < cfg.K ? __fmul_rn(lam32, cfg.bits32[k]) : 0.f;
    build_envelope(cfg, lamb, pr.env);
}

__global__ void alloc_init_kernel(AllocProblem *prob, unsigned long long *acc, int P, int K, const AllocCfg cfg) {
    const int p = blockIdx.x;
    if (threadIdx.x == 0) {
        AllocProblem z = {};
        z.lo = 0.0; z.hi = 1.0; z.lam = 1.0;
        z.phase = K == 1 ? 2 : 0;
        z.sel_level = -1;
        if (z.phase == 0) refresh_envelope(z, cfg);
        prob[p] = z;
    }
    for (int i = threadIdx.x; i < kAccLen; i += blockDim.x) acc[(size_t)p * kAccLen + i] = 0ull;
}

__global__ void alloc_stats_kernel(const float *__restrict__ scores, const uint8_t *__restrict__ sink_mask, int n,
                                   AllocProblem *prob) {
    const int p = blockIdx.y;
    unsigned best = 0;
    int nonfinite = 0, finite = 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        if (sink_mask && sink_mask[i]) continue;
        float s = scores[(size_t)p * n + i];
        if (s != s) { nonfinite = 1; continue; }
        s = fmaxf(s, 0.0f);
        if (isinf(s)) nonfinite = 1;
        else { finite = 1; best = max(best, __float_as_uint(s)); }
    }
    best = __reduce_max_sync(0xffffffffu, best);
    nonfinite = __any_sync(0xffffffffu, nonfinite);
    finite = __any_sync(0xffffffffu, finite);
    if ((threadIdx.x & 31) == 0) {
        if (finite) { atomicMax(&prob[p].max_finite_bits, best); prob[p].any_finite = 1; }
        if (nonfinite) prob[p].any_nonfinite = 1;
    }
}

// next gap-closure pair with something to move; sets phase 3 (select) or 5 (done)
__device__ inline void setup_step(AllocProblem &pr, const AllocCfg &cfg) {
    const int K = cfg.K;
    while (pr.step >= 0 && pr.step <= K - 2) {
        const int lower = pr.step, upper = pr.step + 1;
        const double delta = (double)cfg.bits32[upper] - (double)cfg.bits32[lower];
        if (delta > 0) {
            const int from = pr.dir > 0 ? upper : lower;
            long long want = (long long)(pr.gap / delta + 0.5);
            long long nm = pr.level_counts[from] < want ? pr.level_counts[from] : want;
            if (nm > 0) {
                pr.sel_level = from;
                pr.sel_to = pr.dir > 0 ? lower : upper;
                pr.sel_k = nm;
                pr.n_move = nm;
                pr.sel_prefix = 0ull;
                pr.sel_pass = 0;
                pr.phase = 3;
                return;
            }
        }
        pr.step += pr.dir > 0 ? 1 : -1;
    }
    pr.sel_level = -1;
    pr.phase = 5;
}

// level of one score by the reference's three-operation fp32 cost
__device__ inline int exact_level(float s, const AllocCfg &cfg, const float *lamb) {
    float best = __fadd_rn(__fmul_rn(s, cfg.eps32[0]), lamb[0]);
    int arg = 0;
#pragma unroll
    for (int k = 1; k < kMaxL; ++k) {
        if (k < cfg.K) {
            const float c = __fadd_rn(__fmul_rn(s, cfg.eps32[k]), lamb[k]);
            if (c < best) { best = c; arg = k; }
        }
    }
    return arg;
}

// First index of the ascending keys[0, na) whose score is >= x (upper = false) or > x (upper = true).  Called by a
// whole warp: 32 probes per round, so a million keys take four dependent loads.
__device__ inline int warp_bound(const unsigned *__restrict__ keys, int na, float x, bool upper, int lane) {
    int a = 0, b = na;
    while (b - a > 32) {
        const int step = (b - a + 31) >> 5;
        const int pos = a + lane * step;
        bool go = false;
        if (pos < b) {
            const float kv = __uint_as_float(keys[pos]);
            go = upper ? (kv <= x) : (kv < x);
        }
        const int cnt = __popc(__ballot_sync(0xffffffffu, go));   // the probes answer true ... true false ... false
        if (cnt == 0) { b = a; break; }
        const int nb = a + cnt * step;
        a = a + (cnt - 1) * step + 1;
        if (nb < b) b = nb;
    }
    bool go = false;
    if (a + lane < b) {
        const float kv = __uint_as_float(keys[a + lane]);
        go = upper ? (kv <= x) : (kv < x);
    }
    return a + __popc(__ballot_sync(0xffffffffu, go));
}

// Selection of a gap-closure step from the sorted scores (single-device path; blockDim.x == kAllocThreads).
// The step moves the sel_k candidates of level sel_level with the smallest keys (score, index) -- the largest when
// the direction is "promote".  The level of a score depends on its value only, and the levels of this step's
// candidates are still those of the final assignment (earlier steps moved tokens between other levels), so in the
// ascending order of the scores the candidates are: whole pieces of the cost envelope whose level is sel_level, plus
// the scores inside the bands around the breakpoints for which the three-operation cost says so.  Walking through
// these segments gives the score x of the sel_k-th candidate and the number k' of candidates with exactly that score
// that belong to the selection, which is what two histogram passes over the 32 score bits of the keys find.  When
// every candidate with score x is selected, the index bits need no passes either: the cut is (x, largest index).
// On anything unexpected (no valid envelope, a band of more than 65 536 scores, counts that do not add up) the state
// is left alone and the histogram passes do the selection.
constexpr int kSelMaxExact = 1 << 16;
constexpr int kSelSegs = 2 * kMaxL + 2;

__device__ void sorted_select(AllocProblem *prp, const unsigned *__restrict__ keys, const AllocCfg &cfg) {
    __shared__ Envelope env;
    __shared__ int sg_a[kSelSegs], sg_b[kSelSegs], sg_level[kSelSegs], sg_cnt[kSelSegs];
    __shared__ int sh_edge[2 * kMaxL];
    __shared__ int sh_ns, sh_seg, sh_pos, sh_lb, sh_ub, sh_wsum[kAllocThreads / 32];
    __shared__ long long sh_rem;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int na = prp->n_sorted, L = prp->sel_level;
    const bool inv = prp->dir < 0;
    const long long k = prp->sel_k;
    const float lam32 = (float)prp->lam;
    float lamb[kMaxL];
#pragma unroll
    for (int j = 0; j < kMaxL; ++j) lamb[j] = j < cfg.K ? __fmul_rn(lam32, cfg.bits32[j]) : 0.f;
    if (tid == 0) build_envelope(cfg, lamb, env);
    __syncthreads();
    const int nh = env.nh;
    if (nh == 0 || na <= 0) return;
    for (int e = warp; e < 2 * (nh - 1); e += kAllocThreads / 32) {
        const bool upper = e & 1;
        const int r = warp_bound(keys, na, upper ? env.hi[e >> 1] : env.lo[e >> 1], upper, lane);
        if (lane == 0) sh_edge[e] = r;
    }
    __syncthreads();
    if (tid == 0) {
        int ns = 0, cursor = 0;
        for (int v = 0; v + 1 < nh; ++v) {
            const int i_lo = sh_edge[2 * v], i_hi = sh_edge[2 * v + 1];
            if (i_lo > cursor) {
                sg_a[ns] = cursor; sg_b[ns] = i_lo; sg_level[ns] = env.level[v];
                sg_cnt[ns] = env.level[v] == L ? i_lo - cursor : 0;
                ++ns; cursor = i_lo;
            }
            if (i_hi > cursor) { sg_a[ns] = cursor; sg_b[ns] = i_hi; sg_level[ns] = -1; sg_cnt[ns] = 0; ++ns; cursor = i_hi; }
        }
        if (na > cursor) {
            sg_a[ns] = cursor; sg_b[ns] = na; sg_level[ns] = env.level[nh - 1];
            sg_cnt[ns] = env.level[nh - 1] == L ? na - cursor : 0;
            ++ns;
        }
        sh_ns = ns;
    }
    __syncthreads();
    const int ns = sh_ns;
    for (int sgi = 0; sgi < ns; ++sgi) {
        if (sg_level[sgi] >= 0) continue;
        if (sg_b[sgi] - sg_a[sgi] > kSelMaxExact) return;
        int c = 0;
        for (int i = sg_a[sgi] + tid; i < sg_b[sgi]; i += kAllocThreads) c += exact_level(__uint_as_float(keys[i]), cfg, lamb) == L ? 1 : 0;
        c = __reduce_add_sync(0xffffffffu, c);
        if (lane == 0 && c) atomicAdd(&sg_cnt[sgi], c);
    }
    __syncthreads();
    if (tid == 0) {
        long long rem = k;
        int seg = -1;
        for (int q = 0; q < ns; ++q) {
            const int sgi = inv ? ns - 1 - q : q;
            if (rem <= (long long)sg_cnt[sgi]) { seg = sgi; break; }
            rem -= (long long)sg_cnt[sgi];
        }
        sh_seg = seg;
        sh_rem = rem;
        sh_pos = -1;
        if (seg >= 0 && sg_level[seg] >= 0) sh_pos = inv ? sg_b[seg] - (int)rem : sg_a[seg] + (int)rem - 1;
    }
    __syncthreads();
    const int seg = sh_seg;
    if (seg < 0) return;
    if (sg_level[seg] < 0) {
        // the candidate sits inside a band: walk through it in key order, one block-wide step of 256 scores at a time
        const int a = sg_a[seg], b = sg_b[seg];
        long long rem = sh_rem;
        bool found = false;
        for (int c0 = 0; c0 < b - a; c0 += kAllocThreads) {
            const int off = c0 + tid;
            const int i = inv ? b - 1 - off : a + off;
            const bool hit = off < b - a && exact_level(__uint_as_float(keys[i]), cfg, lamb) == L;
            const unsigned bal = __ballot_sync(0xffffffffu, hit);
            if (lane == 0) sh_wsum[warp] = __popc(bal);
            __syncthreads();
            int before = 0, total = 0;
            for (int w2 = 0; w2 < kAllocThreads / 32; ++w2) {
                if (w2 < warp) before += sh_wsum[w2];
                total += sh_wsum[w2];
            }
            if (rem <= (long long)total) {
                if (hit && before + __popc(bal & ((1u << lane) - 1u)) + 1 == (int)rem) sh_pos = i;
                found = true;
            }
            __syncthreads();
            if (found) break;
            rem -= (long long)total;
        }
        if (!found) return;
    }
    const int pos = sh_pos;
    if (pos < 0 || pos >= na) return;
    const unsigned xb = keys[pos];
    if (warp < 2) {
        const int r = warp_bound(keys, na, __uint_as_float(xb), warp == 1, lane);
        if (lane == 0) { if (warp == 1) sh_ub = r; else sh_lb = r; }
    }
    __syncthreads();
    if (tid == 0) {
        const int lb = sh_lb, ub = sh_ub;
        const long long take = inv ? (long long)(ub - pos) : (long long)(pos - lb + 1);   // of the ub - lb candidates with score x
        const unsigned long long top = inv ? (unsigned long long)(unsigned)(~xb) : (unsigned long long)xb;
        if (take >= 1 && take <= (long long)(ub - lb)) {
            if (take == (long long)(ub - lb)) {
                prp->sel_prefix = (top << 32) | 0xffffffffull;   // all of them: no cut among equal scores
                prp->sel_pass = 4;
                prp->phase = 4;
            } else {
                prp->sel_prefix = top;
                prp->sel_k = take;
                prp->sel_pass = 2;
            }
        }
    }
    __syncthreads();
}

// State update of one problem after a pass; called by a whole block (blockDim.x == kAllocThreads).  With the sorted
// scores of the problem at hand (`keys`), a gap-closure step that has just been set up is resolved from them.
__device__ void update_problem(AllocProblem *prp, unsigned long long *acc, const AllocCfg &cfg, const unsigned *keys = nullptr) {
    __shared__ unsigned long long part[kAllocThreads];
    __shared__ int sh_phase;
    const int tid = threadIdx.x;
    if (tid == 0) sh_phase = prp->phase;
    __syncthreads();
    const int phase = sh_phase;
    if (phase <= 2) {
        if (tid == 0) {
            AllocProblem pr = *prp;
            long long total = 0, nact = 0, counts[kMaxL];
            for (int k = 0; k < cfg.K; ++k) {
                counts[k] = (long long)acc[k];
                total += counts[k] * (long long)cfg.levels[k];
                nact += counts[k];
            }
            const double avg = (double)((float)total / (float)nact);
            pr.evals += 1;
            if (phase == 0) {
                if (avg > cfg.target && pr.hi < 1e8) { pr.hi *= 10.0; pr.lam = pr.hi; }
                else { pr.phase = 1; pr.iter = 0; pr.lam = (pr.lo + pr.hi) * 0.5; }
            } else if (phase == 1) {
                if (avg > cfg.target) pr.lo = pr.lam; else pr.hi = pr.lam;
                pr.iter += 1;
                pr.lam = (pr.lo + pr.hi) * 0.5;
                if (pr.iter == 64) pr.phase = 2;
            }
            if (phase <= 1 && pr.phase <= 1) refresh_envelope(pr, cfg);   // the next pass counts at the new lambda
            if (phase == 2) {
                pr.n_active = (int)nact;
                for (int k = 0; k < cfg.K; ++k) pr.level_counts[k] = counts[k];
                pr.ties_lambda = (int)acc[8];
                double gap = (avg - cfg.target) * (double)nact;
                pr.gap_before = gap;
                if (cfg.K > 1 && fabs(gap) > 0.5) {
                    pr.dir = gap > 0 ? 1 : -1;
                    pr.gap = fabs(gap);
                    pr.step = pr.dir > 0 ? 0 : cfg.K - 2;
                    setup_step(pr, cfg);
                } else {
                    pr.phase = 5;
                }
            }
            *prp = pr;
        }
        if (tid < kAccHead) acc[tid] = 0ull;
    } else if (phase == 3) {
        // find the 16-bit digit holding the sel_k-th smallest key of the current prefix bucket
        unsigned long long *hist = acc + kAccHead;
        const long long k = prp->sel_k;
        const int per = kHistBins / kAllocThreads;
        unsigned long long s = 0;
        for (int i = 0; i < per; ++i) s += hist[tid * per + i];
        part[tid] = s;
        __syncthreads();
        if (tid == 0) {
            unsigned long long run = 0;
            for (int i = 0; i < kAllocThreads; ++i) { unsigned long long v = part[i]; part[i] = run; run += v; }
        }
        __syncthreads();
        const unsigned long long before = part[tid];
        if ((long long)before < k && k <= (long long)(before + s)) {
            unsigned long long run = before;
            for (int i = 0; i < per; ++i) {
                unsigned long long h = hist[tid * per + i];
                if ((long long)run < k && k <= (long long)(run + h)) {
                    AllocProblem pr = *prp;
                    pr.sel_prefix = (pr.sel_prefix << 16) | (unsigned long long)(tid * per + i);
                    pr.sel_k = k - (long long)run;
                    pr.sel_pass += 1;
                    if (pr.sel_pass == 4) pr.phase = 4;
                    *prp = pr;
                    break;
                }
                run += h;
            }
        }
        __syncthreads();
        for (int i = tid; i < kAccLen; i += kAllocThreads) acc[i] = 0ull;
    } else if (phase == 4) {
        if (tid == 0) {
            AllocProblem pr = *prp;
            if (acc[9] > 0 && acc[10] > 0) pr.ties_cut += 1;
            const int lower = pr.step, upper = pr.step + 1;
            const double delta = (double)cfg.bits32[upper] - (double)cfg.bits32[lower];
            pr.moved += (int)pr.n_move;
            pr.level_counts[pr.sel_level] -= pr.n_move;
            pr.level_counts[pr.sel_to] += pr.n_move;
            pr.gap -= (double)pr.n_move * delta;
            if (pr.gap <= 0.5) { pr.phase = 5; pr.sel_level = -1; }
            else { pr.step += pr.dir > 0 ? 1 : -1; setup_step(pr, cfg); }
            *prp = pr;
        }
        if (tid < kAccHead) acc[tid] = 0ull;
    }
    __syncthreads();
    if (keys != nullptr) {
        __shared__ int sh_select;
        if (tid == 0) sh_select = prp->phase == 3 && prp->sel_pass == 0;
        __syncthreads();
        if (sh_select) sorted_select(prp, keys, cfg);
    }
}

__device__ inline unsigned long long make_key(float s, long long gidx, bool invert) {
    unsigned long long key = ((unsigned long long)__float_as_uint(s) << 32) | (unsigned long long)(unsigned)gidx;
    return invert ? ~key : key;
}

// One pass over the scores of every problem.  FUSED: the last block of a problem updates its state.
template <bool FUSED>
__global__ void __launch_bounds__(kAllocThreads, 3) alloc_pass_kernel(const float *__restrict__ scores,
                                                                   const uint8_t *__restrict__ sink_mask, int n,
                                                                   long long idx_base, AllocWs ws, const AllocCfg cfg) {
    __shared__ unsigned long long sh_cnt[kAccHead];
    __shared__ int sh_last;
    __shared__ Envelope sh_env;
    const int p = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    AllocProblem *prp = ws.prob + p;
    unsigned long long *acc = ws.acc + (size_t)p * kAccLen;
    const AllocProblem pr = *prp;   // state is only written between passes
    const int phase = pr.phase;
    if (phase == 5) return;
    const float *sc = scores + (size_t)p * n;
    uint8_t *chosen = ws.chosen + (size_t)p * n;
    if (tid < kAccHead) sh_cnt[tid] = 0ull;
    __syncthreads();
    // a block walks over chunks of kAllocThreads * kPerThread scores with the grid's stride
    constexpr long long kChunk = (long long)kAllocThreads * kPerThread;
    const long long base0 = (long long)blockIdx.x * kChunk, stride = (long long)gridDim.x * kChunk;

    if (phase <= 2) {
        const float lam32 = (float)pr.lam;
        float lamb[kMaxL];
#pragma unroll
        for (int k = 0; k < kMaxL; ++k) lamb[k] = k < cfg.K ? __fmul_rn(lam32, cfg.bits32[k]) : 0.f;
        unsigned cnt[kMaxL];
#pragma unroll
        for (int k = 0; k < kMaxL; ++k) cnt[k] = 0;
        unsigned ties = 0;
        if (phase <= 1) {
            // counting passes: level by envelope breakpoints, full formula only inside the bands
            if (tid == 0) sh_env = prp->env;
            __syncthreads();
            const int nh = sh_env.nh;
            float blo[kMaxL], bhi[kMaxL];
#pragma unroll
            for (int v = 0; v < kMaxL; ++v) {
                blo[v] = v + 1 < nh ? sh_env.lo[v] : INFINITY;
                bhi[v] = v + 1 < nh ? sh_env.hi[v] : INFINITY;
            }
            unsigned long long packed = 0ull;   // eight 8-bit counters, one per envelope piece or level
            int since_flush = 0;
            // software pipeline: the loads of the next chunk are in flight while this one is counted
            float sv_n[kPerThread];
            int mk_n[kPerThread];
            auto load_chunk = [&](long long base) {
#pragma unroll
                for (int u = 0; u < kPerThread; ++u) {
                    const long long i = base + u * kAllocThreads + tid;
                    const bool in = i < n;
                    sv_n[u] = in ? __ldg(sc + i) : 0.f;
                    mk_n[u] = in ? (sink_mask ? (int)__ldg(sink_mask + i) : 0) : -1;
                }
            };
            if (base0 < n) load_chunk(base0);
            for (long long base = base0; base < n; base += stride) {
                float sv[kPerThread];
                int mk[kPerThread];
#pragma unroll
                for (int u = 0; u < kPerThread; ++u) { sv[u] = sv_n[u]; mk[u] = mk_n[u]; }
                if (base + stride < n) load_chunk(base + stride);
                // branch-free for the eight scores; the few that sit inside a band are redone below
                unsigned redo = 0;
#pragma unroll
                for (int u = 0; u < kPerThread; ++u) {
                    const float s = sanitize(sv[u], pr);
                    sv[u] = s;
                    int above = 0, reached = 0;
#pragma unroll
                    for (int v = 0; v < kMaxL - 1; ++v) { above += (s > bhi[v]) ? 1 : 0; reached += (s >= blo[v]) ? 1 : 0; }
                    const bool live = mk[u] == 0;
                    const bool sure = nh > 0 && above == reached;
                    const int arg = sh_env.level[above];
                    packed += (live && sure) ? (1ull << (8 * arg)) : 0ull;
                    redo |= (live && !sure) ? (1u << u) : 0u;
                }
                while (redo) {
                    const int u = __ffs(redo) - 1;
                    redo &= redo - 1;
                    float s = 0.f;
#pragma unroll
                    for (int uu = 0; uu < kPerThread; ++uu) s = uu == u ? sv[uu] : s;
                    float best = __fadd_rn(__fmul_rn(s, cfg.eps32[0]), lamb[0]);
                    int arg = 0;
#pragma unroll
                    for (int k = 1; k < kMaxL; ++k) {
                        if (k < cfg.K) {
                            float c = __fadd_rn(__fmul_rn(s, cfg.eps32[k]), lamb[k]);
                            if (c < best) { best = c; arg = k; }
                        }
                    }
                    packed += 1ull << (8 * arg);
                }
                if (++since_flush == 31) {
#pragma unroll
                    for (int k = 0; k < kMaxL; ++k) cnt[k] += (unsigned)((packed >> (8 * k)) & 0xffull);
                    packed = 0ull;
                    since_flush = 0;
                }
            }
#pragma unroll
            for (int k = 0; k < kMaxL; ++k) cnt[k] += (unsigned)((packed >> (8 * k)) & 0xffull);
        } else
        for (long long base = base0; base < n; base += stride) {
            // all loads of the iteration are issued before the first one is used
            float sv[kPerThread];
            int mk[kPerThread];
#pragma unroll
            for (int u = 0; u < kPerThread; ++u) {
                const long long i = base + u * kAllocThreads + tid;
                const bool in = i < n;
                sv[u] = in ? sc[i] : 0.f;
                mk[u] = in ? (sink_mask ? (int)sink_mask[i] : 0) : -1;
            }
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            long long i = base + u * kAllocThreads + tid;
            if (mk[u] < 0) continue;
            if (mk[u]) { if (phase == 2) chosen[i] = 255; continue; }
            const float s = sanitize(sv[u], pr);
            float best = __fadd_rn(__fmul_rn(s, cfg.eps32[0]), lamb[0]);
            float cost[kMaxL];
            cost[0] = best;
            int arg = 0;
#pragma unroll
            for (int k = 1; k < kMaxL; ++k) {
                if (k < cfg.K) {
                    float c = __fadd_rn(__fmul_rn(s, cfg.eps32[k]), lamb[k]);
                    cost[k] = c;
                    if (c < best) { best = c; arg = k; }
                }
            }
#pragma unroll
            for (int k = 0; k < kMaxL; ++k) cnt[k] += (arg == k);
            if (phase == 2) {
                chosen[i] = (uint8_t)arg;
#pragma unroll
                for (int k = 0; k < kMaxL; ++k) {
                    if (k == arg) {
                        if (k >= 1 && fabs((double)cost[k - 1] - (double)cost[k]) < 1e-6) ties++;
                        if (k + 1 < cfg.K && fabs((double)cost[k] - (double)cost[k + 1 < kMaxL ? k + 1 : k]) < 1e-6) ties++;
                    }
                }
            }
        }
        }
#pragma unroll
        for (int k = 0; k < kMaxL; ++k) {
            unsigned v = __reduce_add_sync(0xffffffffu, cnt[k]);
            if (lane == 0 && v) atomicAdd(&sh_cnt[k], (unsigned long long)v);
        }
        unsigned tv = __reduce_add_sync(0xffffffffu, ties);
        if (lane == 0 && tv) atomicAdd(&sh_cnt[8], (unsigned long long)tv);
        __syncthreads();
        if (tid < kAccHead && sh_cnt[tid]) atomicAdd(&acc[tid], sh_cnt[tid]);
    } else if (phase == 3) {
        const bool inv = pr.dir < 0;
        const int shift_digit = 48 - 16 * pr.sel_pass;
        for (long long base = base0; base < n; base += stride) {
            float sv[kPerThread];
            int ch[kPerThread];
#pragma unroll
            for (int u = 0; u < kPerThread; ++u) {
                const long long i = base + u * kAllocThreads + tid;
                const bool in = i < n;
                sv[u] = in ? sc[i] : 0.f;
                ch[u] = in ? (int)chosen[i] : -1;
            }
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            long long i = base + u * kAllocThreads + tid;
            if (ch[u] != (int)(uint8_t)pr.sel_level) continue;
            unsigned long long key = make_key(sanitize(sv[u], pr), idx_base + i, inv);
            if (pr.sel_pass > 0 && (key >> (shift_digit + 16)) != pr.sel_prefix) continue;
            atomicAdd(&acc[kAccHead + ((key >> shift_digit) & 0xffffull)], 1ull);
        }
        }
    } else {  // phase 4: move every candidate whose key is <= the selected key
        const bool inv = pr.dir < 0;
        const unsigned long long cut = pr.sel_prefix;
        const unsigned cut_score = (unsigned)((inv ? ~cut : cut) >> 32);
        unsigned same_sel = 0, same_unsel = 0;
        for (long long base = base0; base < n; base += stride) {
            float sv[kPerThread];
            int ch[kPerThread];
#pragma unroll
            for (int u = 0; u < kPerThread; ++u) {
                const long long i = base + u * kAllocThreads + tid;
                const bool in = i < n;
                sv[u] = in ? sc[i] : 0.f;
                ch[u] = in ? (int)chosen[i] : -1;
            }
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            long long i = base + u * kAllocThreads + tid;
            if (ch[u] != (int)(uint8_t)pr.sel_level) continue;
            const float s = sanitize(sv[u], pr);
            unsigned long long key = make_key(s, idx_base + i, inv);
            const bool sel = key <= cut;
            if (sel) chosen[i] = (uint8_t)pr.sel_to;
            if (__float_as_uint(s) == cut_score) { if (sel) same_sel++; else same_unsel++; }
        }
        }
        unsigned a = __reduce_add_sync(0xffffffffu, same_sel), b = __reduce_add_sync(0xffffffffu, same_unsel);
        if (lane == 0) {
            if (a) atomicAdd(&acc[9], (unsigned long long)a);
            if (b) atomicAdd(&acc[10], (unsigned long long)b);
        }
    }

    if (FUSED) {
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            unsigned t = atomicAdd(&prp->ticket, 1u);
            sh_last = (t == gridDim.x - 1);
        }
        __syncthreads();
        if (sh_last) {
            __threadfence();
            if (tid == 0) prp->ticket = 0;
            update_problem(prp, acc, cfg, cfg.K > 1 ? ws.keys_out + (size_t)p * n : nullptr);   // this form runs after the sort
        }
    }
}

// ---- sorted-score solver for the counting passes (single-device path) -----------------------------------
// The scores of a problem are sorted once (keys = bit patterns of the sanitised, non-negative scores; sinks sort
// to the end).  A counting pass at a given lambda then needs, per breakpoint band of the envelope, two binary
// searches and the exact evaluation of the few scores inside the band; everything between two bands belongs to
// one envelope piece.  One CTA per problem runs all widening and bisection steps back to back.
__global__ void alloc_keys_kernel(const float *__restrict__ scores, const uint8_t *__restrict__ sink_mask, int n, AllocWs ws) {
    const int p = blockIdx.y;
    const AllocProblem pr = ws.prob[p];
    unsigned live = 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const bool sink = sink_mask && sink_mask[i];
        ws.keys_in[(size_t)p * n + i] = sink ? 0xffffffffu : __float_as_uint(sanitize(scores[(size_t)p * n + i], pr));
        live += sink ? 0u : 1u;
    }
    live = __reduce_add_sync(0xffffffffu, live);
    if ((threadIdx.x & 31) == 0 && live) atomicAdd(&ws.prob[p].n_sorted, (int)live);
}

constexpr int kSolveThreads = 512;
constexpr int kCoarse = 4096;

__global__ void __launch_bounds__(kSolveThreads) alloc_solve_kernel(AllocWs ws, int n, const AllocCfg cfg) {
    __shared__ float coarse[kCoarse];
    __shared__ unsigned sh_counts[kMaxL];
    __shared__ int sh_edge[2 * kMaxL];      // per band: first index >= lo, first index > hi
    __shared__ int sh_rng[2 * kMaxL + 2];   // exact ranges [start, end)
    __shared__ int sh_nr, sh_phase;
    const int p = blockIdx.x, tid = threadIdx.x;
    // the problem's state and its 16 counters live in shared memory for the whole solve (some 66 dependent steps, each
    // of which would otherwise wait for several round trips to global memory) and go back at the end
    __shared__ AllocProblem pr_s;
    __shared__ unsigned long long acc_s[kAccHead];
    AllocProblem *const prp_g = ws.prob + p;
    unsigned long long *const acc_g = ws.acc + (size_t)p * kAccLen;
    if (tid == 0) pr_s = *prp_g;
    if (tid < kAccHead) acc_s[tid] = acc_g[tid];
    __syncthreads();
    AllocProblem *prp = &pr_s;
    unsigned long long *acc = acc_s;
    const unsigned *keys = ws.keys_out + (size_t)p * n;
    const int na = prp->n_sorted;
    const int stride = na > kCoarse ? (na + kCoarse - 1) / kCoarse : 1;
    const int nc = na > 0 ? (na + stride - 1) / stride : 0;
    for (int i = tid; i < nc; i += kSolveThreads) coarse[i] = __uint_as_float(keys[(size_t)i * stride]);
    if (tid == 0) sh_phase = prp->phase;
    __syncthreads();
    for (int guard = 0; guard < kEvalRounds + 2 && sh_phase <= 1; ++guard) {
        const float lam32 = (float)prp->lam;
        float lamb[kMaxL];
#pragma unroll
        for (int k = 0; k < kMaxL; ++k) lamb[k] = k < cfg.K ? __fmul_rn(lam32, cfg.bits32[k]) : 0.f;
        const int nh = prp->env.nh;
        if (tid < kMaxL) sh_counts[tid] = 0;
        // ---- band edges: one warp per edge; coarse index in shared memory, then the stride around it is narrowed
        //      by 32 probes at a time (two dependent loads for a stride of 256 instead of eight)
        if (nh > 1 && (tid >> 5) < 2 * (nh - 1)) {
            const int w = tid >> 5, lane = tid & 31;
            const int v = w >> 1;
            const bool upper = w & 1;
            const float x = upper ? prp->env.hi[v] : prp->env.lo[v];
            int lo = 0, hi = nc;   // first coarse entry that is >= x (lower) or > x (upper)
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                const bool go = upper ? (coarse[mid] <= x) : (coarse[mid] < x);
                if (go) lo = mid + 1; else hi = mid;
            }
            int a = lo > 0 ? (lo - 1) * stride : 0, b = lo < nc ? lo * stride : na;
            if (b > na) b = na;
            // the edge (first key that is not "before x") lies in [a, b]; keys are sorted, so the probes answer
            // true ... true false ... false
            while (b - a > 32) {
                const int step = (b - a + 31) >> 5;
                const int pos = a + lane * step;
                bool go = false;
                if (pos < b) {
                    const float kv = __uint_as_float(keys[pos]);
                    go = upper ? (kv <= x) : (kv < x);
                }
                const int cnt = __popc(__ballot_sync(0xffffffffu, go));
                if (cnt == 0) { b = a; break; }
                const int nb = a + cnt * step;
                a = a + (cnt - 1) * step + 1;
                if (nb < b) b = nb;
            }
            {
                bool go = false;
                if (a + lane < b) {
                    const float kv = __uint_as_float(keys[a + lane]);
                    go = upper ? (kv <= x) : (kv < x);
                }
                a += __popc(__ballot_sync(0xffffffffu, go));
            }
            if (lane == 0) sh_edge[w] = a;
        }
        __syncthreads();
        // ---- pieces between the bands and the exact ranges inside them
        if (tid == 0) {
            int nr = 0, cursor = 0;
            if (nh == 0) { sh_rng[0] = 0; sh_rng[1] = na; nr = 1; cursor = na; }
            for (int v = 0; v + 1 < nh; ++v) {
                const int i_lo = sh_edge[2 * v], i_hi = sh_edge[2 * v + 1];
                if (i_lo > cursor) { sh_counts[prp->env.level[v]] += (unsigned)(i_lo - cursor); cursor = i_lo; }
                if (i_hi > cursor) { sh_rng[2 * nr] = cursor; sh_rng[2 * nr + 1] = i_hi; ++nr; cursor = i_hi; }
            }
            if (nh > 0 && na > cursor) sh_counts[prp->env.level[nh - 1]] += (unsigned)(na - cursor);
            sh_nr = nr;
        }
        __syncthreads();
        for (int r = 0; r < sh_nr; ++r) {
            for (int i = sh_rng[2 * r] + tid; i < sh_rng[2 * r + 1]; i += kSolveThreads) {
                const float sc = __uint_as_float(keys[i]);
                float best = __fadd_rn(__fmul_rn(sc, cfg.eps32[0]), lamb[0]);
                int arg = 0;
#pragma unroll
                for (int k = 1; k < kMaxL; ++k) {
                    if (k < cfg.K) {
                        const float c = __fadd_rn(__fmul_rn(sc, cfg.eps32[k]), lamb[k]);
                        if (c < best) { best = c; arg = k; }
                    }
                }
                atomicAdd(&sh_counts[arg], 1u);
            }
        }
        __syncthreads();
        if (tid < kMaxL) acc[tid] = (unsigned long long)sh_counts[tid];
        __syncthreads();
        update_problem(prp, acc, cfg);   // advances lo / hi / lambda and the envelope exactly as a fused pass does
        if (tid == 0) sh_phase = prp->phase;
        __syncthreads();
    }
    if (tid == 0) *prp_g = pr_s;
    if (tid < kAccHead) acc_g[tid] = acc_s[tid];
}

// blocks per problem of a pass: enough to fill the GPU a few times over, never more than one chunk each
static int pass_blocks(int n, int P) {
    const int chunks = (n + kAllocThreads * kPerThread - 1) / (kAllocThreads * kPerThread);
    int want = (6 * 148 + P - 1) / P;
    if (want < 1) want = 1;
    return chunks < want ? chunks : want;
}

// stepwise path: copy the accumulator out / consume the rank-summed accumulator
__global__ void alloc_export_acc_kernel(const unsigned long long *__restrict__ acc, long long *__restrict__ exchange, int len) {
    const int p = blockIdx.y;
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < len) exchange[(size_t)p * len + i] = (long long)acc[(size_t)p * kAccLen + i];
}
__global__ void __launch_bounds__(kAllocThreads) alloc_update_kernel(AllocWs ws, const long long *__restrict__ reduced, int len,
                                                                      const AllocCfg cfg) {
    const int p = blockIdx.x;
    unsigned long long *acc = ws.acc + (size_t)p * kAccLen;
    for (int i = threadIdx.x; i < len; i += blockDim.x) acc[i] = (unsigned long long)reduced[(size_t)p * len + i];
    __syncthreads();
    update_problem(ws.prob + p, acc, cfg);
}

__global__ void alloc_emit_kernel(const uint8_t *__restrict__ sink_mask, int n, AllocWs ws, const AllocCfg cfg,
                                  int32_t *__restrict__ bits, odmkv_alloc_report *__restrict__ reports) {
    const int p = blockIdx.y;
    const uint8_t *chosen = ws.chosen + (size_t)p * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        uint8_t c = chosen[i];
        bits[(size_t)p * n + i] = (c == 255 || (sink_mask && sink_mask[i])) ? cfg.sink_bits : cfg.levels[c < kMaxL ? c : 0];
    }
    if (reports && blockIdx.x == 0 && threadIdx.x == 0) {
        const AllocProblem &pr = ws.prob[p];
        odmkv_alloc_report r = {};
        r.lam = pr.lam;
        r.gap_before = pr.gap_before;
        for (int k = 0; k < kMaxL; ++k) r.counts[k] = k < cfg.K ? pr.level_counts[k] : 0;
        r.n_active = pr.n_active;
        r.evaluations = pr.evals;
        r.moved = pr.moved;
        r.ties_lambda = pr.ties_lambda;
        r.ties_cut = pr.ties_cut;
        r.done = pr.phase == 5;
        reports[p] = r;
    }
}

static int make_cfg(const int *levels, const double *eps, int K, double target, int sink_bits, AllocCfg *cfg) {
    if (!levels || !eps) return ODMKV_ERR_ARG;
    if (K < 1 || K > kMaxL) return ODMKV_ERR_LIMIT;
    for (int k = 0; k < K; ++k) {
        if (k > 0 && levels[k] <= levels[k - 1]) return ODMKV_ERR_ARG;
        cfg->levels[k] = levels[k];
        cfg->bits32[k] = (float)levels[k];
        cfg->eps32[k] = (float)eps[k];
    }
    for (int k = K; k < kMaxL; ++k) { cfg->levels[k] = 0; cfg->bits32[k] = 0.f; cfg->eps32[k] = 0.f; }
    for (int i = 0; i < kMaxL; ++i)
        for (int j = 0; j < kMaxL; ++j) {
            const double d = (double)cfg->eps32[i] - (double)cfg->eps32[j];
            cfg->inv_da[i * kMaxL + j] = d != 0.0 ? 1.0 / d : 0.0;
        }
    cfg->K = K;
    cfg->sink_bits = sink_bits;
    double t = target;
    if (t < (double)levels[0]) t = (double)levels[0];
    if (t > (double)levels[K - 1]) t = (double)levels[K - 1];
    cfg->target = t;
    return ODMKV_OK;
}

// Helper streams on which the sorts of different problems run side by side (a sort of 1 M keys is five short
// kernels that leave most of the GPU idle).  Created on the first call on a device (host objects, no device memory);
// that call must not be made while a stream is being captured.
struct SortLanes { cudaStream_t stream[kSortLanes]; cudaEvent_t fork, join[kSortLanes]; bool ok; };
static SortLanes *sort_lanes() {
    static SortLanes table[64] = {};
    static bool tried[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!tried[dev]) {
        tried[dev] = true;
        SortLanes &l = table[dev];
        bool ok = cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) == cudaSuccess;
        for (int j = 0; j < kSortLanes && ok; ++j)
            ok = cudaStreamCreateWithFlags(&l.stream[j], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&l.join[j], cudaEventDisableTiming) == cudaSuccess;
        l.ok = ok;
    }
    return table[dev].ok ? &table[dev] : nullptr;
}

static inline int closure_rounds(int K) { return K > 1 ? 5 * (K - 1) : 0; }

// host-side mirror of what a stepwise caller needs between calls
struct AllocHostCtx {
    AllocHeader hdr;
    AllocCfg cfg;
    int round;
};

}  // namespace odmkv

using namespace odmkv;

extern "C" {

size_t odmkv_alloc_workspace_bytes(int P, int n) {
    if (P <= 0 || n <= 0) return 0;
    return alloc_ws_layout(P, n, nullptr, nullptr) + 256;
}

static int alloc_begin_impl(const float *scores, const uint8_t *sink_mask, int P, int n, const AllocCfg &cfg, AllocWs *ws,
                            void *workspace, size_t workspace_bytes, cudaStream_t st) {
    if (!scores || !workspace) return ODMKV_ERR_ARG;
    if (P <= 0 || n <= 0 || P > 65535) return ODMKV_ERR_SHAPE;
    if (((uintptr_t)workspace & 255) != 0) return ODMKV_ERR_WORKSPACE;
    if (workspace_bytes < alloc_ws_layout(P, n, ws, (unsigned char *)workspace)) return ODMKV_ERR_WORKSPACE;
    alloc_init_kernel<<<P, 256, 0, st>>>(ws->prob, ws->acc, P, cfg.K, cfg);
    int blocks = (n + 256 * 8 - 1) / (256 * 8);
    if (blocks > 1024) blocks = 1024;
    alloc_stats_kernel<<<dim3(blocks, P), 256, 0, st>>>(scores, sink_mask, n, ws->prob);
    return launch_status();
}

int odmkv_allocate_bits(const float *scores, const uint8_t *sink_mask, int P, int n, const int *levels,
                        const double *eps, int K, double target_avg_bits, int sink_bits, int32_t *bits,
                        odmkv_alloc_report *reports, void *workspace, size_t workspace_bytes, void *stream) {
    if (!bits) return ODMKV_ERR_ARG;
    AllocCfg cfg;
    int rc = make_cfg(levels, eps, K, target_avg_bits, sink_bits, &cfg);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    AllocWs ws;
    rc = alloc_begin_impl(scores, sink_mask, P, n, cfg, &ws, workspace, workspace_bytes, st);
    if (rc) return rc;
    const int nblk = pass_blocks(n, P);
    const int rounds = 1 + closure_rounds(K);   // the final assignment pass and the gap closure
    timing_begin("allocate", st);
    if (K > 1) {
        int kb = (n + 256 * 8 - 1) / (256 * 8);
        if (kb > 1024) kb = 1024;
        alloc_keys_kernel<<<dim3(kb, P), 256, 0, st>>>(scores, sink_mask, n, ws);
        // problem p is sorted on lane p % kSortLanes (its own stream and slice of the scratch); the lanes start after
        // the keys are written and the caller's stream goes on when all of them are done
        SortLanes *lanes = P > 1 ? sort_lanes() : nullptr;
        const int nl = lanes ? (P < kSortLanes ? P : kSortLanes) : 0;
        if (lanes) {
            cudaError_t e = cudaEventRecord(lanes->fork, st);
            for (int j = 0; j < nl && e == cudaSuccess; ++j) e = cudaStreamWaitEvent(lanes->stream[j], lanes->fork, 0);
            if (e != cudaSuccess) return (int)e;
        }
        for (int p = 0; p < P; ++p) {
            const int j = lanes ? p % kSortLanes : 0;
            size_t tb = ws.sort_temp_bytes;
            cudaError_t e = cub::DeviceRadixSort::SortKeys((unsigned char *)ws.sort_temp + (size_t)j * ws.sort_temp_bytes, tb,
                                                           ws.keys_in + (size_t)p * n, ws.keys_out + (size_t)p * n, n, 0, 32,
                                                           lanes ? lanes->stream[j] : st);
            if (e != cudaSuccess) return (int)e;
        }
        for (int j = 0; j < nl; ++j) {
            cudaError_t e = cudaEventRecord(lanes->join[j], lanes->stream[j]);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(st, lanes->join[j], 0);
            if (e != cudaSuccess) return (int)e;
        }
        alloc_solve_kernel<<<P, kSolveThreads, 0, st>>>(ws, n, cfg);
    }
    for (int r = 0; r < rounds; ++r)
        alloc_pass_kernel<true><<<dim3(nblk, P), kAllocThreads, 0, st>>>(scores, sink_mask, n, 0ll, ws, cfg);
    timing_end(st);
    int eb = (n + 255) / 256;
    if (eb > 2048) eb = 2048;
    alloc_emit_kernel<<<dim3(eb, P), 256, 0, st>>>(sink_mask, n, ws, cfg, bits, reports);
    return launch_status();
}

// ---- stepwise (rank-sharded) form ------------------------------------------------------------
// The workspace starts with a small host-readable header region that this library only writes
// from the host side through cudaMemcpyAsync; the per-call context lives in a static table keyed
// by the workspace pointer so that eval/update/finish need no extra arguments.
}  // extern "C"

#include <map>
#include <mutex>
namespace odmkv {
static std::mutex g_ctx_mu;
static std::map<void *, AllocHostCtx> g_ctx;
}  // namespace odmkv

extern "C" {

size_t odmkv_alloc_exchange_len(void) { return (size_t)kAccLen; }
int odmkv_alloc_num_rounds(int K) { return K > 1 ? kEvalRounds + closure_rounds(K) : 1; }

int odmkv_alloc_begin(const float *scores, const uint8_t *sink_mask, int P, int n_local, long long idx_base,
                      const int *levels, const double *eps, int K, double target_avg_bits, int sink_bits,
                      void *workspace, size_t workspace_bytes, long long *exchange, void *stream) {
    if (!exchange) return ODMKV_ERR_ARG;
    AllocHostCtx ctx;
    int rc = make_cfg(levels, eps, K, target_avg_bits, sink_bits, &ctx.cfg);
    if (rc) return rc;
    AllocWs ws;
    rc = alloc_begin_impl(scores, sink_mask, P, n_local, ctx.cfg, &ws, workspace, workspace_bytes, (cudaStream_t)stream);
    if (rc) return rc;
    ctx.hdr.scores = scores; ctx.hdr.sink_mask = sink_mask; ctx.hdr.P = P; ctx.hdr.n = n_local; ctx.hdr.idx_base = idx_base;
    ctx.round = 0;
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    g_ctx[workspace] = ctx;
    return ODMKV_OK;
}

static int get_ctx(void *workspace, AllocHostCtx *out, AllocWs *ws) {
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    auto it = g_ctx.find(workspace);
    if (it == g_ctx.end()) return ODMKV_ERR_ARG;
    *out = it->second;
    alloc_ws_layout(out->hdr.P, out->hdr.n, ws, (unsigned char *)workspace);
    return ODMKV_OK;
}

int odmkv_alloc_eval(void *workspace, long long *exchange, void *stream) {
    AllocHostCtx ctx; AllocWs ws;
    int rc = get_ctx(workspace, &ctx, &ws);
    if (rc) return rc;
    if (!exchange) return ODMKV_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int n = ctx.hdr.n, P = ctx.hdr.P;
    const int nblk = pass_blocks(n, P);
    alloc_pass_kernel<false><<<dim3(nblk, P), kAllocThreads, 0, st>>>(ctx.hdr.scores, ctx.hdr.sink_mask, n, ctx.hdr.idx_base, ws, ctx.cfg);
    alloc_export_acc_kernel<<<dim3((kAccLen + 255) / 256, P), 256, 0, st>>>(ws.acc, exchange, kAccLen);
    return launch_status();
}

int odmkv_alloc_update(void *workspace, const long long *exchange_reduced, void *stream) {
    AllocHostCtx ctx; AllocWs ws;
    int rc = get_ctx(workspace, &ctx, &ws);
    if (rc) return rc;
    if (!exchange_reduced) return ODMKV_ERR_ARG;
    alloc_update_kernel<<<ctx.hdr.P, kAllocThreads, 0, (cudaStream_t)stream>>>(ws, exchange_reduced, kAccLen, ctx.cfg);
    return launch_status();
}

int odmkv_alloc_finish(void *workspace, int32_t *bits, odmkv_alloc_report *reports, void *stream) {
    AllocHostCtx ctx; AllocWs ws;
    int rc = get_ctx(workspace, &ctx, &ws);
    if (rc) return rc;
    if (!bits) return ODMKV_ERR_ARG;
    const int n = ctx.hdr.n;
    int eb = (n + 255) / 256;
    if (eb > 2048) eb = 2048;
    alloc_emit_kernel<<<dim3(eb, ctx.hdr.P), 256, 0, (cudaStream_t)stream>>>(ctx.hdr.sink_mask, n, ws, ctx.cfg, bits, reports);
    {
        std::lock_guard<std::mutex> lk(g_ctx_mu);
        g_ctx.erase(workspace);
    }
    return launch_status();
}

}  // extern "C"
