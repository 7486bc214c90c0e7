// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the decode path: a serving loop whose memory
// pool is frozen after start-up, a real-time thread that may not take the driver's allocation lock, or
// a plug-in that is handed raw device pointers and owns no allocator at all.  The regular entry points
// ask such callers for a workspace they have no way to obtain.  This file gives them one entry point
// whose scratch lives in a file-scope __device__ array instead.
//
// Consequences the caller has to know:
//   * every GPU that loads the library holds the array (kNoAllocScratchBytes) until the process exits;
//   * sizes whose partials do not fit are rejected with ODMKV_ERR_LIMIT, nothing is launched;
//   * the first call on each device looks the array's device address up (cudaGetSymbolAddress), and the first
//     decode call on a device creates a helper stream and two events and sets the kernels' shared-memory
//     attribute (host objects, no device memory); make that first call before starting any stream capture;
//   * all calls on a device share the array and it keeps the previous call's contents.  Nothing in it
//     has to start at zero: every partial slot a call reads is written by that same call first.  Two
//     calls that overlap on the GPU (different streams) would race on it -- issue them on one stream.
#include "decode_shared.cuh"

namespace odmkv {

constexpr size_t kNoAllocScratchBytes = 6u << 20;   // 6 MiB: e.g. 64 (sample, KV head) pairs x 16 partial slots x 8 heads
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// In host code the array's name is only a handle; the address the kernels need comes from the runtime,
// once per device, with that device current.
static unsigned char *g_scratch_addr[kMaxDevices] = {};

static int scratch_for_current_device(unsigned char **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return ODMKV_ERR_LIMIT;
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_addr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_scratch_addr[dev];
    return ODMKV_OK;
}

}  // namespace odmkv

using namespace odmkv;

extern "C" {

int odmkv_decode_attn_mma(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                          const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                          const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                          int out_dtype, float *lse, int n_splits, void *workspace, size_t workspace_bytes,
                          const float *lut_scales, void *stream);

size_t odmkv_decode_attn_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

int odmkv_decode_attn_noalloc(const void *q, int q_dtype, const odmkv_chunk *chunks, int n_chunks, int cache_dtype,
                              const void *tail_k, const void *tail_v, int tail_len, int tail_cap, const float *pi_k,
                              const float *pi_v, const float *codebooks, int B, int H, int G, float scale, void *out,
                              int out_dtype, float *lse, int n_splits, const float *lut_scales, void *stream) {
    if (B <= 0 || H <= 0 || G <= 0 || G > 8 || n_splits <= 0 || n_splits > 128) return ODMKV_ERR_SHAPE;
    // the tensor-core launcher adds up to 8 partial slots for exact / tail tokens
    if (decode_ws_layout(B, H, G, n_splits + 8, nullptr, nullptr) > kNoAllocScratchBytes) return ODMKV_ERR_LIMIT;
    unsigned char *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    return odmkv_decode_attn_mma(q, q_dtype, chunks, n_chunks, cache_dtype, tail_k, tail_v, tail_len, tail_cap, pi_k, pi_v, codebooks,
                                 B, H, G, scale, out, out_dtype, lse, n_splits, scratch, kNoAllocScratchBytes, lut_scales, stream);
}

}  // extern "C"
