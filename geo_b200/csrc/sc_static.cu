// SC conv2d forward for callers that cannot hand the library a workspace.
//
// Some hosts of this library have no way to obtain device memory at the point where they call
// it: code running under a framework's memory planner that has already sized and frozen its
// pools, a real-time inference loop that is forbidden to touch the allocator after start-up, or a
// plugin boundary that passes only tensor pointers and no allocator handle.  For them the stream
// scratch (packed activation streams, packed weight streams, member offset table) lives in one
// fixed array inside the library image instead of in a caller-owned buffer.
//
// The price of that convenience: every GPU that loads the library carries the array for the life
// of the process, problems whose scratch exceeds it are refused, and because all calls share the
// one array, two calls whose kernels could overlap on the GPU (different streams, different host
// threads) would overwrite each other's streams -- the caller must serialise them.
#include <mutex>

#include "sc_common.h"

namespace geo {

// 64 MiB: enough for every layer of the 4-layer SC CNN at batch 256 with 128-bit streams
// (largest: 32x20x20 padded input, 52.4 MB of activation streams + 0.8 MB of weight streams).
constexpr size_t kStaticScratchBytes = 64ull << 20;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel
// could use; the device address is looked up once per device and cached here.
static std::mutex g_static_mutex;
static void *g_static_ptr[64] = {};

static int static_scratch(void **ptr) {
    int dev = 0;
    GEO_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(GEO_SC_ERR_UNSUPPORTED, "device index %d", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);  // the current device's copy
        if (e != cudaSuccess || !p)
            return fail(GEO_SC_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        g_static_ptr[dev] = p;
    }
    *ptr = g_static_ptr[dev];
    return GEO_SC_OK;
}

}  // namespace geo

using namespace geo;

extern "C" {

size_t geo_sc_static_scratch_bytes(void) { return kStaticScratchBytes; }

int geo_sc_conv2d_forward_static(const geo_sc_conv_desc *desc, const float *act, const float *weight, int32_t *out,
                                 void *stream) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!act || !weight || !out) return fail(GEO_SC_ERR_NULL, "act, weight or out is NULL");
    const size_t ab = align_up(g.act_stream_words * 4, 256);
    const size_t wb = align_up(g.w_stream_words * 4, 256);
    const size_t tb = align_up(g.aoff_entries * 4, 256);
    if (ab + wb + tb > kStaticScratchBytes)
        return fail(GEO_SC_ERR_WORKSPACE,
                    "this convolution needs %zu bytes of stream scratch but the built-in scratch holds %zu; "
                    "split the batch or use geo_sc_conv2d_forward with a caller-owned workspace",
                    ab + wb + tb, kStaticScratchBytes);
    void *base = nullptr;
    if ((rc = static_scratch(&base))) return rc;
    uint32_t *as = (uint32_t *)base;
    uint32_t *ws = (uint32_t *)((char *)base + ab);
    int32_t *aoff = (int32_t *)((char *)base + ab + wb);
    cudaStream_t s = (cudaStream_t)stream;
    // Every word of the three regions is rewritten by the two generation kernels before the
    // accumulation kernel reads it, so nothing left over from an earlier call can leak in; the
    // output is cleared inside launch_accumulate whenever it is accumulated into.
    if ((rc = launch_prepare_weights(g, weight, ws, aoff, s))) return rc;
    if ((rc = launch_act_streams(g, act, as, s))) return rc;
    return launch_accumulate(g, as, ws, aoff, out, s);
}

}  // extern "C"
