// Process-wide plumbing of libqutai_moe.so: error text, launch counters, per-kernel-class event
// timing, the device status word, and the small memory/stream helpers of the C ABI.
#include <atomic>
#include <map>
#include <mutex>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <vector>

#include "common.cuh"

namespace qmoe {

namespace {
thread_local char g_error[1024] = "";
std::atomic<long long> g_launches{0};
std::atomic<long long> g_tc_launches{0};
bool g_sync_each_launch = getenv("QUTAI_MOE_SYNC") && atoi(getenv("QUTAI_MOE_SYNC")) != 0;

// timing
std::mutex g_timing_mutex;
bool g_timing = false;
struct Scope { int kc; cudaEvent_t start, stop; };
std::vector<Scope> g_scopes;
const char* kClassNames[KC_COUNT] = {"router_gemm", "route", "permute", "expert_gemm", "swiglu", "combine",
                                     "combine_backward", "wgrad_gemm", "unpermute", "route_backward",
                                     "cast", "other", "exchange", "optimizer", "norm", "attention", "head_loss",
                                     "elementwise", "barrier", "all_reduce"};
__device__ int g_device_status;
std::atomic<int> g_variants[QMOE_VARIANT_COUNT];  // zero-initialised: every kernel in its default form
}  // namespace

int kernel_variant(int which) { return g_variants[which].load(std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail_arg(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return QMOE_ERR_ARGUMENT;
}

int check_cuda(cudaError_t code, const char* what) {
    if (code == cudaSuccess) return 0;
    set_error("%s failed: %s (%s)", what, cudaGetErrorName(code), cudaGetErrorString(code));
    return (int)code;
}

int after_launch(const char* name) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t code = cudaGetLastError();
    if (code == cudaSuccess && g_sync_each_launch) code = cudaDeviceSynchronize();
    if (code == cudaSuccess) return 0;
    set_error("kernel %s failed: %s (%s)", name, cudaGetErrorName(code), cudaGetErrorString(code));
    return (int)code;
}

void count_tensor_core_launch() { g_tc_launches.fetch_add(1, std::memory_order_relaxed); }

}  // namespace qmoe

extern "C" int qmoe_test_select_variant(int32_t which, int32_t value) {
    if (which < 0 || which >= QMOE_VARIANT_COUNT) return qmoe::fail_arg("test_select_variant: unknown selector %d", which);
    if (value < 0 || value > 1) return qmoe::fail_arg("test_select_variant: value must be 0 (default) or 1");
    qmoe::g_variants[which].store(value, std::memory_order_relaxed);
    return 0;
}

namespace qmoe {

int* device_status_address() {
    int* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_device_status) != cudaSuccess) return nullptr;
    return p;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

TimedScope::TimedScope(KernelClass kc, cudaStream_t s) : slot(-1), stream(s) {
    if (!g_timing) return;
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    Scope sc;
    sc.kc = kc;
    if (cudaEventCreate(&sc.start) != cudaSuccess) return;
    if (cudaEventCreate(&sc.stop) != cudaSuccess) { cudaEventDestroy(sc.start); return; }
    cudaEventRecord(sc.start, stream);
    g_scopes.push_back(sc);
    slot = (int)g_scopes.size() - 1;
}

TimedScope::~TimedScope() {
    if (slot < 0) return;
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    if (slot < (int)g_scopes.size()) cudaEventRecord(g_scopes[slot].stop, stream);
}

}  // namespace qmoe

using namespace qmoe;

extern "C" int qmoe_version(void) { return QMOE_VERSION; }
extern "C" const char* qmoe_last_error(void) { return g_error; }

extern "C" int qmoe_device_info(int* sms, int* cc_major, int* cc_minor, uint64_t* total_bytes) {
    int dev = 0;
    QMOE_CUDA(cudaGetDevice(&dev));
    cudaDeviceProp prop;
    QMOE_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (sms) *sms = prop.multiProcessorCount;
    if (cc_major) *cc_major = prop.major;
    if (cc_minor) *cc_minor = prop.minor;
    if (total_bytes) *total_bytes = (uint64_t)prop.totalGlobalMem;
    return 0;
}

extern "C" int qmoe_malloc(uint64_t* address, uint64_t bytes) {
    if (!address) return fail_arg("malloc: address is null");
    void* p = nullptr;
    QMOE_CUDA(cudaMalloc(&p, bytes ? bytes : 1));
    *address = (uint64_t)p;
    return 0;
}
extern "C" int qmoe_free(uint64_t address) {
    if (!address) return 0;
    QMOE_CUDA(cudaFree((void*)address));
    return 0;
}
extern "C" int qmoe_host_alloc(void** host, uint64_t bytes) {
    if (!host) return fail_arg("host_alloc: host is null");
    QMOE_CUDA(cudaMallocHost(host, bytes ? bytes : 1));
    return 0;
}
extern "C" int qmoe_host_free(void* host) {
    if (!host) return 0;
    QMOE_CUDA(cudaFreeHost(host));
    return 0;
}
extern "C" int qmoe_memcpy_h2d(uint64_t dst, const void* src, uint64_t bytes, uint64_t stream) {
    if (!bytes) return 0;
    if (!dst || !src) return fail_arg("memcpy_h2d: null address");
    QMOE_CUDA(cudaMemcpyAsync((void*)dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return 0;
}
extern "C" int qmoe_memcpy_d2h(void* dst, uint64_t src, uint64_t bytes, uint64_t stream) {
    if (!bytes) return 0;
    if (!dst || !src) return fail_arg("memcpy_d2h: null address");
    QMOE_CUDA(cudaMemcpyAsync(dst, (const void*)src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return 0;
}
extern "C" int qmoe_memcpy_d2d(uint64_t dst, uint64_t src, uint64_t bytes, uint64_t stream) {
    if (!bytes) return 0;
    if (!dst || !src) return fail_arg("memcpy_d2d: null address");
    QMOE_CUDA(cudaMemcpyAsync((void*)dst, (const void*)src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return 0;
}
extern "C" int qmoe_memset(uint64_t dst, int value, uint64_t bytes, uint64_t stream) {
    if (!bytes) return 0;
    if (!dst) return fail_arg("memset: null address");
    QMOE_CUDA(cudaMemsetAsync((void*)dst, value, bytes, (cudaStream_t)stream));
    return 0;
}
extern "C" int qmoe_stream_sync(uint64_t stream) {
    QMOE_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return 0;
}
extern "C" int64_t qmoe_launch_count(void) { return g_launches.load(); }
extern "C" int64_t qmoe_tensor_core_launch_count(void) { return g_tc_launches.load(); }

extern "C" int qmoe_timing_enable(int enable) {
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    for (auto& s : g_scopes) { cudaEventDestroy(s.start); cudaEventDestroy(s.stop); }
    g_scopes.clear();
    g_timing = enable != 0;
    return 0;
}
extern "C" int qmoe_timing_classes(void) { return KC_COUNT; }
extern "C" const char* qmoe_timing_class_name(int kc) { return kc >= 0 && kc < KC_COUNT ? kClassNames[kc] : ""; }
extern "C" int qmoe_timing_read(double* ms, int64_t* scopes, int capacity) {
    if (!ms || !scopes || capacity < KC_COUNT) return fail_arg("timing_read: need %d slots", KC_COUNT);
    QMOE_CUDA(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    for (int i = 0; i < KC_COUNT; ++i) { ms[i] = 0; scopes[i] = 0; }
    for (auto& s : g_scopes) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, s.start, s.stop) == cudaSuccess) { ms[s.kc] += t; scopes[s.kc] += 1; }
    }
    return 0;
}

extern "C" int qmoe_device_status(uint64_t stream, int* status) {
    if (!status) return fail_arg("device_status: status is null");
    int* p = device_status_address();
    if (!p) { set_error("device status symbol is not available"); return QMOE_ERR_STATE; }
    QMOE_CUDA(cudaMemcpyAsync(status, p, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    QMOE_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return 0;
}

extern "C" int qmoe_device_status_async(uint64_t stream, void* host_status) {
    if (!host_status) return fail_arg("device_status_async: host_status is null");
    int* p = device_status_address();
    if (!p) { set_error("device status symbol is not available"); return QMOE_ERR_STATE; }
    QMOE_CUDA(cudaMemcpyAsync(host_status, p, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return 0;
}

// ---- streams and events for hosts that overlap transfers or exchanges with compute -------------
extern "C" int qmoe_stream_create(uint64_t* stream) {
    if (!stream) return fail_arg("stream_create: stream is null");
    cudaStream_t s = nullptr;
    QMOE_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = (uint64_t)s;
    return 0;
}
extern "C" int qmoe_stream_destroy(uint64_t stream) {
    if (!stream) return 0;
    QMOE_CUDA(cudaStreamDestroy((cudaStream_t)stream));
    return 0;
}
extern "C" int qmoe_event_create(uint64_t* event) {
    if (!event) return fail_arg("event_create: event is null");
    cudaEvent_t e = nullptr;
    QMOE_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    *event = (uint64_t)e;
    return 0;
}
extern "C" int qmoe_event_destroy(uint64_t event) {
    if (!event) return 0;
    QMOE_CUDA(cudaEventDestroy((cudaEvent_t)event));
    return 0;
}
extern "C" int qmoe_event_record(uint64_t event, uint64_t stream) {
    if (!event) return fail_arg("event_record: event is null");
    QMOE_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return 0;
}
extern "C" int qmoe_stream_wait_event(uint64_t stream, uint64_t event) {
    if (!event) return fail_arg("stream_wait_event: event is null");
    QMOE_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
    return 0;
}
extern "C" int qmoe_event_sync(uint64_t event) {
    if (!event) return fail_arg("event_sync: event is null");
    QMOE_CUDA(cudaEventSynchronize((cudaEvent_t)event));
    return 0;
}
// ---- CUDA graphs: a launch-bound sequence (the decode-shaped forward: about ten short kernels) recorded
// once and replayed with one call -----------------------------------------------------------------------
namespace {
std::mutex g_graph_mutex;
std::map<uint64_t, long long> g_graph_kernels;        // kernels recorded in each instantiated graph
thread_local long long g_capture_started_at = 0;      // launch counter when this thread's capture began
}  // namespace

extern "C" int qmoe_graph_begin(uint64_t stream) {
    if (!stream) return fail_arg("graph_begin: capture needs a stream of its own, not the default stream");
    if (g_sync_each_launch) { set_error("graph capture is not possible with QUTAI_MOE_SYNC=1"); return QMOE_ERR_STATE; }
    QMOE_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    g_capture_started_at = g_launches.load();
    return 0;
}
extern "C" int qmoe_graph_end(uint64_t stream, uint64_t* graph) {
    if (!graph) return fail_arg("graph_end: graph is null");
    *graph = 0;
    cudaGraph_t recorded = nullptr;
    QMOE_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &recorded));
    cudaGraphExec_t exec = nullptr;
    cudaError_t code = cudaGraphInstantiate(&exec, recorded, 0);
    cudaGraphDestroy(recorded);
    QMOE_CUDA(code);
    *graph = (uint64_t)exec;
    const long long recorded_kernels = g_launches.load() - g_capture_started_at;
    g_launches.fetch_sub(recorded_kernels, std::memory_order_relaxed);  // they were recorded, not run
    std::lock_guard<std::mutex> lock(g_graph_mutex);
    g_graph_kernels[*graph] = recorded_kernels;
    return 0;
}
extern "C" int qmoe_graph_abandon(uint64_t stream) {  // after a failed call during capture: end it, drop the result
    cudaGraph_t recorded = nullptr;
    cudaStreamEndCapture((cudaStream_t)stream, &recorded);
    if (recorded) cudaGraphDestroy(recorded);
    cudaGetLastError();
    return 0;
}
extern "C" int qmoe_graph_launch(uint64_t graph, uint64_t stream) {
    if (!graph) return fail_arg("graph_launch: graph is null");
    QMOE_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph, (cudaStream_t)stream));
    long long kernels = 1;
    {
        std::lock_guard<std::mutex> lock(g_graph_mutex);
        auto it = g_graph_kernels.find(graph);
        if (it != g_graph_kernels.end()) kernels = it->second;
    }
    g_launches.fetch_add(kernels, std::memory_order_relaxed);  // the launch counter counts kernels that ran
    return 0;
}
extern "C" int qmoe_graph_destroy(uint64_t graph) {
    if (!graph) return 0;
    QMOE_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph));
    std::lock_guard<std::mutex> lock(g_graph_mutex);
    g_graph_kernels.erase(graph);
    return 0;
}

extern "C" int qmoe_device_status_clear(uint64_t stream) {
    int* p = device_status_address();
    if (!p) { set_error("device status symbol is not available"); return QMOE_ERR_STATE; }
    QMOE_CUDA(cudaMemsetAsync(p, 0, sizeof(int), (cudaStream_t)stream));
    return 0;
}
