// Per-device runtime state of the library: the host-visible status word that device-side waits report to,
// and the library-owned scratch of the kernels that hand data over through global memory.
//
// The reference keeps its per-device state in `Device` (stream, cuBLAS handle, module cache:
// xn-core/src/cuda_backend.rs:35-60) and turns every CUDA failure into an Err (xn-core/src/error.rs:71-92).
// Here a kernel cannot return an error, so a wait that ran out increments one 32-bit word per device that
// lives in pinned, mapped host memory: the host reads it without synchronising, every later launch on that
// device is refused with XN_ERR_DEVICE until xn_mm_clear_device_status(), and xn_mm_device_status() lets a
// caller poll it at its own synchronisation points.
#include <mutex>
#include <vector>

#include "common.cuh"
#include <nvtx3/nvToolsExt.h>
#include "wait.cuh"

namespace xn {

static bool nvtx_enabled() {
    static const bool on = [] { const char *e = getenv("XN_MM_NVTX"); return e && atoi(e) != 0; }();
    return on;
}
ApiRange::ApiRange(const char *name) : on(nvtx_enabled()) {
    if (on) nvtxRangePushA(name);
}
ApiRange::~ApiRange() {
    if (on) nvtxRangePop();
}

namespace {

constexpr int MAX_DEV = 64;
std::mutex g_mu;
volatile unsigned *g_status[MAX_DEV];  // host-mapped status words (one page-locked word per device)

struct StreamScratch {
    int dev;
    cudaStream_t st;
    SkinnyScratch s;
};
std::vector<StreamScratch> g_table;
// Blocks that were replaced by larger ones.  A block may have been baked into a captured graph or be in use
// by a launch another host thread is about to enqueue, so it is never freed behind the caller's back: it
// stays here until xn_mm_release_scratch().
struct Retired { int dev; void *p; };
std::vector<Retired> g_retired;

thread_local bool tl_no_alloc = false;

int current_device(int *dev) {
    XN_CHECK_CUDA(cudaGetDevice(dev));
    if (*dev < 0 || *dev >= MAX_DEV) return fail(XN_ERR_UNSUPPORTED, "device index %d outside the library's table", *dev);
    return XN_OK;
}

__global__ void selftest_wait_kernel(WaitCtx w, unsigned *gave_up) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((unsigned)__cvta_generic_to_shared(&bar)), "r"(1u));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // nobody ever arrives on `bar`: the wait has to run out, report, and let the kernel finish normally
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait_bounded((unsigned)__cvta_generic_to_shared(&bar), 0u, w);
        if (gave_up) *gave_up = ok ? 0u : 1u;
    }
}

}  // namespace

NoAllocScope::NoAllocScope() : prev(tl_no_alloc) { tl_no_alloc = true; }
NoAllocScope::~NoAllocScope() { tl_no_alloc = prev; }

int wait_ctx(WaitCtx *out) {
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    out->limit_ns = WAIT_LIMIT_NS;
    volatile unsigned *w = g_status[dev];
    if (!w) {
        if (tl_no_alloc) {  // the allocation-free entry point: the waits stay bounded, the report is skipped
            out->status = nullptr;
            return XN_OK;
        }
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_status[dev]) {
            void *p = nullptr;
            XN_CHECK_CUDA(cudaHostAlloc(&p, 64, cudaHostAllocMapped | cudaHostAllocPortable));
            *static_cast<volatile unsigned *>(p) = 0;
            g_status[dev] = static_cast<volatile unsigned *>(p);
        }
        w = g_status[dev];
    }
    const unsigned n = *w;
    if (n)
        return fail(XN_ERR_DEVICE,
                    "%u device-side wait(s) ran out in an earlier launch on device %d: results since then are undefined; "
                    "synchronise, recover, then call xn_mm_clear_device_status()", n, dev);
    void *dp = nullptr;
    XN_CHECK_CUDA(cudaHostGetDevicePointer(&dp, const_cast<unsigned *>(w), 0));
    out->status = static_cast<unsigned *>(dp);
    return XN_OK;
}

// Scratch of the skinny path (partial accumulators + arrival counters) and of the f32 repack: one buffer per
// (device, stream), allocated when a stream first needs it and replaced by a larger one on demand.  Calls on one
// stream are ordered, so they can share; calls on different streams get different buffers and may overlap.
// (xn drives a device through one stream, xn-core/src/cuda_backend.rs:52: one buffer per GPU in practice.)
// A stream that is being captured cannot allocate: it borrows the largest buffer of its device -- the one of the
// stream that ran the same shapes before the capture, which is how a CUDA graph is normally warmed up -- and is
// refused with a clear message when no buffer is large enough.
int skinny_scratch(cudaStream_t st, size_t partial_bytes, size_t ncounters, SkinnyScratch *out) {
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    XN_CHECK_CUDA(cudaStreamIsCapturing(st, &cap));
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    std::lock_guard<std::mutex> lock(g_mu);
    StreamScratch *e = nullptr;
    for (auto &t : g_table)
        if (t.dev == dev && t.st == st) { e = &t; break; }
    if (capturing) {
        if (!e || e->s.partial_bytes < partial_bytes || e->s.ncounters < ncounters) {
            e = nullptr;
            for (auto &t : g_table)
                if (t.dev == dev && t.s.partial_bytes >= partial_bytes && t.s.ncounters >= ncounters &&
                    (!e || t.s.partial_bytes > e->s.partial_bytes))
                    e = &t;
        }
        if (!e)
            return fail(XN_ERR_UNSUPPORTED,
                        "this shape needs %zu bytes of library scratch and the stream is being captured; "
                        "run the call once outside stream capture first", partial_bytes);
        *out = e->s;
        return XN_OK;
    }
    if (!e) {
        g_table.push_back(StreamScratch{dev, st, SkinnyScratch()});
        e = &g_table.back();
    }
    SkinnyScratch &s = e->s;
    if (s.partial_bytes < partial_bytes) {
        void *p = nullptr;
        XN_CHECK_CUDA(cudaMalloc(&p, partial_bytes));
        if (s.partials) g_retired.push_back(Retired{dev, s.partials});
        s.partials = static_cast<float *>(p);
        s.partial_bytes = partial_bytes;
    }
    if (s.ncounters < ncounters) {
        void *p = nullptr;
        XN_CHECK_CUDA(cudaMalloc(&p, ncounters * sizeof(unsigned)));
        // the counters must read zero before the first launch that uses them: ordered on the caller's stream
        XN_CHECK_CUDA(cudaMemsetAsync(p, 0, ncounters * sizeof(unsigned), st));
        if (s.counters) g_retired.push_back(Retired{dev, s.counters});
        s.counters = static_cast<unsigned *>(p);
        s.ncounters = ncounters;
    }
    *out = s;
    return XN_OK;
}

// The same per-(device, stream) buffer for other internal users (the f32 matmul's packed operands).
int library_scratch(cudaStream_t st, size_t bytes, void **out) {
    SkinnyScratch s;
    if (int rc = skinny_scratch(st, bytes, 0, &s)) return rc;
    *out = s.partials;
    return XN_OK;
}

}  // namespace xn

using namespace xn;

extern "C" int xn_mm_device_status(unsigned *timeouts_out) {
    XN_API_RANGE("xn_mm_device_status");
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    volatile unsigned *w = g_status[dev];
    const unsigned n = w ? *w : 0u;
    if (timeouts_out) *timeouts_out = n;
    if (n) return fail(XN_ERR_DEVICE, "%u device-side wait(s) ran out on device %d", n, dev);
    return XN_OK;
}

extern "C" int xn_mm_clear_device_status(void) {
    XN_API_RANGE("xn_mm_clear_device_status");
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    XN_CHECK_CUDA(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_status[dev]) *g_status[dev] = 0;
    // a launch that gave up may have left arrival counters of split tiles non-zero
    for (auto &t : g_table)
        if (t.dev == dev && t.s.counters) XN_CHECK_CUDA(cudaMemset(t.s.counters, 0, t.s.ncounters * sizeof(unsigned)));
    return XN_OK;
}

extern "C" int xn_mm_release_scratch(void *stream, int all_streams) {
    XN_API_RANGE("xn_mm_release_scratch");
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    XN_CHECK_CUDA(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(g_mu);
    for (size_t i = 0; i < g_table.size();) {
        StreamScratch &t = g_table[i];
        if (t.dev == dev && (all_streams || t.st == (cudaStream_t)stream)) {
            if (t.s.partials) XN_CHECK_CUDA(cudaFree(t.s.partials));
            if (t.s.counters) XN_CHECK_CUDA(cudaFree(t.s.counters));
            g_table.erase(g_table.begin() + i);
        } else {
            ++i;
        }
    }
    for (size_t i = 0; i < g_retired.size();) {
        if (g_retired[i].dev == dev) {
            XN_CHECK_CUDA(cudaFree(g_retired[i].p));
            g_retired.erase(g_retired.begin() + i);
        } else {
            ++i;
        }
    }
    return XN_OK;
}

extern "C" int xn_mm_selftest_wait_timeout(unsigned long long limit_ns, void *stream) {
    XN_API_RANGE("xn_mm_selftest_wait_timeout");
    WaitCtx w;
    if (int rc = wait_ctx(&w)) return rc;
    XN_REQUIRE(limit_ns > 0 && limit_ns <= WAIT_LIMIT_NS, "selftest: limit_ns=%llu outside (0, %llu]", limit_ns, WAIT_LIMIT_NS);
    w.limit_ns = limit_ns;
    selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(w, nullptr);
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}
