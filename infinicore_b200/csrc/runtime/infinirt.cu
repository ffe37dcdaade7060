// libinfinirt: the runtime C API over the CUDA runtime, NVIDIA devices only.
//
// Mirrors the behaviour of reference src/infinirt/infinirt.cc (dispatcher, thread-local
// current device) and src/infinirt/cuda/infinirt_cuda.cu:264-470 (CUDA backend) for the
// entry points declared in include/infinirt.h.  There is no CPU backend: with the
// current device left at INFINI_DEVICE_CPU (the initial state of every thread) all
// stream/event/memory calls return INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED.
#include "infinirt.h"

#include <cstring>
#include <cuda_runtime.h>

#include <cstdio>
#include <chrono>
#include <cstdlib>
#include <deque>
#include <dlfcn.h>
#include <memory>
#include <mutex>
#include <utility>
#include <vector>

namespace {

thread_local infiniDevice_t t_device_type = INFINI_DEVICE_CPU;
thread_local int t_device_id = 0;

inline infiniStatus_t fromCuda(cudaError_t err, const char *what) {
    if (err == cudaSuccess) {
        return INFINI_STATUS_SUCCESS;
    }
    std::fprintf(stderr, "[infinirt] %s failed: %s\n", what, cudaGetErrorString(err));
    return INFINI_STATUS_INTERNAL_ERROR;
}

#define RT_CUDA(call) return fromCuda((call), #call)

#define RT_REQUIRE_NVIDIA()                                   \
    do {                                                      \
        if (t_device_type != INFINI_DEVICE_NVIDIA) {          \
            return INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED;   \
        }                                                     \
    } while (0)

#define RT_REQUIRE_PTR(p)                                     \
    do {                                                      \
        if ((p) == nullptr) {                                 \
            return INFINI_STATUS_NULL_POINTER;                \
        }                                                     \
    } while (0)

inline cudaMemcpyKind toCudaKind(infinirtMemcpyKind_t kind) {
    switch (kind) {
    case INFINIRT_MEMCPY_H2H:
        return cudaMemcpyHostToHost;
    case INFINIRT_MEMCPY_H2D:
        return cudaMemcpyHostToDevice;
    case INFINIRT_MEMCPY_D2H:
        return cudaMemcpyDeviceToHost;
    case INFINIRT_MEMCPY_D2D:
        return cudaMemcpyDeviceToDevice;
    }
    return cudaMemcpyDefault;
}

} // namespace

__INFINI_C infiniStatus_t infinirtInit() {
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinirtGetDeviceCount(infiniDevice_t device, int *count) {
    RT_REQUIRE_PTR(count);
    if (device == INFINI_DEVICE_CPU) {
        *count = 1;
        return INFINI_STATUS_SUCCESS;
    }
    if (device != INFINI_DEVICE_NVIDIA) {
        *count = 0;
        return INFINI_STATUS_SUCCESS;
    }
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    *count = n;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinirtGetAllDeviceCount(int *count_array) {
    RT_REQUIRE_PTR(count_array);
    for (int i = 0; i < INFINI_DEVICE_TYPE_COUNT; ++i) {
        infiniStatus_t st = infinirtGetDeviceCount(static_cast<infiniDevice_t>(i), &count_array[i]);
        if (st != INFINI_STATUS_SUCCESS) {
            return st;
        }
    }
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinirtSetDevice(infiniDevice_t device, int device_id) {
    if (device == INFINI_DEVICE_CPU) {
        t_device_type = device;
        t_device_id = device_id;
        return INFINI_STATUS_SUCCESS;
    }
    if (device != INFINI_DEVICE_NVIDIA) {
        return INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED;
    }
    cudaError_t err = cudaSetDevice(device_id);
    if (err != cudaSuccess) {
        (void)cudaGetLastError();
        std::fprintf(stderr, "[infinirt] cudaSetDevice(%d) failed: %s\n", device_id, cudaGetErrorString(err));
        return INFINI_STATUS_DEVICE_NOT_FOUND;
    }
    t_device_type = device;
    t_device_id = device_id;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinirtGetDevice(infiniDevice_t *device_ptr, int *device_id_ptr) {
    if (device_ptr == nullptr && device_id_ptr == nullptr) {
        return INFINI_STATUS_NULL_POINTER;
    }
    if (device_ptr != nullptr) {
        *device_ptr = t_device_type;
    }
    if (device_id_ptr != nullptr) {
        *device_id_ptr = t_device_id;
    }
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinirtGetMemInfo(infiniDevice_t device, int device_id, size_t *free_bytes, size_t *total_bytes) {
    RT_REQUIRE_PTR(free_bytes);
    RT_REQUIRE_PTR(total_bytes);
    if (device != INFINI_DEVICE_NVIDIA) {
        return INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED;
    }
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess) {
        return INFINI_STATUS_INTERNAL_ERROR;
    }
    if (cudaSetDevice(device_id) != cudaSuccess) {
        (void)cudaGetLastError();
        return INFINI_STATUS_DEVICE_NOT_FOUND;
    }
    cudaError_t err = cudaMemGetInfo(free_bytes, total_bytes);
    (void)cudaSetDevice(prev);
    return fromCuda(err, "cudaMemGetInfo");
}

// ---- utilisation figures from the driver's management library --------------------------------------------
// The snapshot's utilisation members (reference src/infinirt/cuda/infinirt_cuda.cu:163-262) come from NVML,
// which is not linked: it is looked up at run time (dlopen), only its read-only queries are used, and a
// machine without it simply leaves those members' bits clear.  The device is found by its PCI bus id, so the
// figures belong to the CUDA device asked about whatever CUDA_VISIBLE_DEVICES does to the numbering.
// INFINIRT_MANAGEMENT_LIBRARY names another library to load instead (the tests put a stand-in there).
namespace {

struct Utilization {
    unsigned int gpu;    // percent of the last sample period in which a kernel was running
    unsigned int memory; // percent in which device memory was being read or written
};

class ManagementLibrary {
public:
    static ManagementLibrary &get() {
        static ManagementLibrary lib;
        return lib;
    }

    bool utilization(const char *pci_bus_id, Utilization *out) {
        std::lock_guard<std::mutex> lock(mutex_);
        if (!ready()) {
            return false;
        }
        void *device = nullptr;
        if (by_bus_id_(pci_bus_id, &device) != 0 || device == nullptr) {
            return false;
        }
        return rates_(device, out) == 0;
    }

private:
    using InitFn = int (*)();
    using ByBusIdFn = int (*)(const char *, void **);
    using RatesFn = int (*)(void *, Utilization *);

    ManagementLibrary() {
        const char *override_path = std::getenv("INFINIRT_MANAGEMENT_LIBRARY");
        const char *names[] = {override_path, "libnvidia-ml.so.1", "libnvidia-ml.so"};
        for (const char *name : names) {
            if (name == nullptr || *name == '\0') {
                continue;
            }
            handle_ = dlopen(name, RTLD_LAZY | RTLD_LOCAL);
            if (handle_ != nullptr || name == override_path) {
                break; // a named stand-in that does not load is not replaced by the real thing
            }
        }
        if (handle_ == nullptr) {
            return;
        }
        init_ = reinterpret_cast<InitFn>(dlsym(handle_, "nvmlInit_v2"));
        by_bus_id_ = reinterpret_cast<ByBusIdFn>(dlsym(handle_, "nvmlDeviceGetHandleByPciBusId_v2"));
        rates_ = reinterpret_cast<RatesFn>(dlsym(handle_, "nvmlDeviceGetUtilizationRates"));
    }

    bool ready() {
        if (init_ == nullptr || by_bus_id_ == nullptr || rates_ == nullptr) {
            return false;
        }
        if (!initialised_) {
            initialised_ = (init_() == 0); // stays initialised for the life of the process
        }
        return initialised_;
    }

    std::mutex mutex_;
    void *handle_ = nullptr;
    InitFn init_ = nullptr;
    ByBusIdFn by_bus_id_ = nullptr;
    RatesFn rates_ = nullptr;
    bool initialised_ = false;
};

} // namespace

// ---- communication samples ------------------------------------------------------------------------------
// One ledger per device: event pairs in flight, and the samples that completed during the last second.
namespace {

constexpr int kLedgerDevices = 64;
constexpr double kWindowSeconds = 1.0;

struct EventPair {
    cudaEvent_t start = nullptr;
    cudaEvent_t end = nullptr;
};

struct OpenSample { // what infinirtCommunicationBegin hands out
    EventPair events;
    int device = 0;
};

struct Finished {
    std::chrono::steady_clock::time_point when;
    double ms;
    uint64_t bytes;
};

struct Ledger {
    std::mutex mutex;
    std::vector<EventPair> spare;                      // event pairs ready for reuse
    std::vector<std::pair<EventPair, uint64_t>> inflight; // end event recorded, not yet seen complete
    std::deque<Finished> window;
};

Ledger &ledgerOf(int device) {
    static Ledger ledgers[kLedgerDevices];
    return ledgers[(device >= 0 && device < kLedgerDevices) ? device : 0];
}

// Moves completed samples into the window and drops what is older than the window.  Device `device` is current.
void collectFinished(Ledger &ledger) {
    const auto now = std::chrono::steady_clock::now();
    size_t keep = 0;
    for (size_t i = 0; i < ledger.inflight.size(); ++i) {
        auto &entry = ledger.inflight[i];
        const cudaError_t q = cudaEventQuery(entry.first.end);
        if (q == cudaErrorNotReady) {
            ledger.inflight[keep++] = entry;
            continue;
        }
        float ms = 0.f;
        if (q == cudaSuccess && cudaEventElapsedTime(&ms, entry.first.start, entry.first.end) == cudaSuccess) {
            ledger.window.push_back({now, static_cast<double>(ms), entry.second});
            ledger.spare.push_back(entry.first);
        } else {
            (void)cudaGetLastError(); // an event that cannot be read (e.g. its stream was destroyed): drop the pair
            (void)cudaEventDestroy(entry.first.start);
            (void)cudaEventDestroy(entry.first.end);
        }
    }
    ledger.inflight.resize(keep);
    while (!ledger.window.empty() && std::chrono::duration<double>(now - ledger.window.front().when).count() > kWindowSeconds) {
        ledger.window.pop_front();
    }
}

} // namespace

__INFINI_C infiniStatus_t infinirtCommunicationBegin(infinirtStream_t stream, void **sample) {
    RT_REQUIRE_PTR(sample);
    *sample = nullptr;
    // (the CUDA runtime's current device counts here, whether or not the thread went through infinirtSetDevice:
    // a collective library may be driven by a host framework that selects devices itself)
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
        (void)cudaGetLastError();
        return INFINI_STATUS_SUCCESS; // a graph being recorded: its replays are not sampled
    }
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        (void)cudaGetLastError();
        return INFINI_STATUS_SUCCESS;
    }
    Ledger &ledger = ledgerOf(device);
    EventPair pair;
    {
        std::lock_guard<std::mutex> lock(ledger.mutex);
        if (!ledger.spare.empty()) {
            pair = ledger.spare.back();
            ledger.spare.pop_back();
        }
    }
    if (pair.start == nullptr) {
        if (cudaEventCreate(&pair.start) != cudaSuccess || cudaEventCreate(&pair.end) != cudaSuccess) {
            (void)cudaGetLastError();
            if (pair.start != nullptr) {
                (void)cudaEventDestroy(pair.start);
            }
            return INFINI_STATUS_SUCCESS; // sampling is best effort: the collective itself must not fail over it
        }
    }
    if (cudaEventRecord(pair.start, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        (void)cudaGetLastError();
        std::lock_guard<std::mutex> lock(ledger.mutex);
        ledger.spare.push_back(pair);
        return INFINI_STATUS_SUCCESS;
    }
    *sample = new OpenSample{pair, device};
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinirtCommunicationEnd(void *sample, infinirtStream_t stream, uint64_t bytes) {
    if (sample == nullptr) {
        return INFINI_STATUS_SUCCESS;
    }
    std::unique_ptr<OpenSample> open(static_cast<OpenSample *>(sample));
    Ledger &ledger = ledgerOf(open->device);
    const bool recorded = bytes > 0 && cudaEventRecord(open->events.end, static_cast<cudaStream_t>(stream)) == cudaSuccess;
    if (!recorded) {
        (void)cudaGetLastError();
    }
    std::lock_guard<std::mutex> lock(ledger.mutex);
    if (recorded) {
        ledger.inflight.emplace_back(open->events, bytes);
    } else {
        ledger.spare.push_back(open->events);
    }
    return INFINI_STATUS_SUCCESS;
}

// Memory capacity from the CUDA runtime; compute and memory-bandwidth utilisation from the management library
// when it is there (kernel_time_ratio is the same sample, marked as an estimate, as in the reference); payload
// bytes and time share of the collectives that completed during the last second from the device's ledger.
__INFINI_C infiniStatus_t infinirtGetDeviceResourceSnapshot(infiniDevice_t device, int device_id,
                                                           infinirtDeviceResourceSnapshot_t *snapshot) {
    RT_REQUIRE_PTR(snapshot);
    std::memset(snapshot, 0, sizeof(*snapshot));
    snapshot->device_type = device;
    snapshot->device_id = device_id;
    size_t free_bytes = 0, total_bytes = 0;
    const infiniStatus_t st = infinirtGetMemInfo(device, device_id, &free_bytes, &total_bytes);
    if (st != INFINI_STATUS_SUCCESS) {
        return st;
    }
    snapshot->free_bytes = free_bytes;
    snapshot->total_bytes = total_bytes;
    snapshot->used_bytes = total_bytes - free_bytes;
    snapshot->valid_fields = INFINIRT_RESOURCE_FIELD_MEMORY_CAPACITY;

    char bus_id[32] = {};
    if (cudaDeviceGetPCIBusId(bus_id, static_cast<int>(sizeof(bus_id)), device_id) == cudaSuccess) {
        Utilization u{};
        if (ManagementLibrary::get().utilization(bus_id, &u)) {
            snapshot->compute_utilization = static_cast<float>(u.gpu) / 100.0f;
            snapshot->memory_bandwidth_utilization = static_cast<float>(u.memory) / 100.0f;
            snapshot->kernel_time_ratio = snapshot->compute_utilization;
            snapshot->valid_fields |= INFINIRT_RESOURCE_FIELD_COMPUTE_UTILIZATION | INFINIRT_RESOURCE_FIELD_MEMORY_BANDWIDTH_UTILIZATION
                                      | INFINIRT_RESOURCE_FIELD_KERNEL_TIME_RATIO;
            snapshot->estimated_fields |= INFINIRT_RESOURCE_FIELD_KERNEL_TIME_RATIO;
        }
    } else {
        (void)cudaGetLastError();
    }

    // the ledger's events belong to `device_id`: make it current while they are queried
    int previous = -1;
    if (cudaGetDevice(&previous) == cudaSuccess && (previous == device_id || cudaSetDevice(device_id) == cudaSuccess)) {
        Ledger &ledger = ledgerOf(device_id);
        std::lock_guard<std::mutex> lock(ledger.mutex);
        collectFinished(ledger);
        double ms = 0.0;
        uint64_t bytes = 0;
        for (const Finished &f : ledger.window) {
            ms += f.ms;
            bytes += f.bytes;
        }
        const double ratio = ms / (kWindowSeconds * 1000.0);
        snapshot->communication_bytes = bytes;
        snapshot->communication_time_ratio = static_cast<float>(ratio > 1.0 ? 1.0 : ratio);
        snapshot->valid_fields |= INFINIRT_RESOURCE_FIELD_COMMUNICATION;
        if (previous != device_id) {
            (void)cudaSetDevice(previous);
        }
    } else {
        (void)cudaGetLastError();
    }
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinirtDeviceSynchronize() {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaDeviceSynchronize());
}

// ---- streams -------------------------------------------------------------------------

__INFINI_C infiniStatus_t infinirtStreamCreate(infinirtStream_t *stream_ptr) {
    RT_REQUIRE_PTR(stream_ptr);
    RT_REQUIRE_NVIDIA();
    cudaStream_t s = nullptr;
    cudaError_t err = cudaStreamCreate(&s);
    *stream_ptr = s;
    return fromCuda(err, "cudaStreamCreate");
}

__INFINI_C infiniStatus_t infinirtStreamDestroy(infinirtStream_t stream) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
}

__INFINI_C infiniStatus_t infinirtStreamSynchronize(infinirtStream_t stream) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
}

__INFINI_C infiniStatus_t infinirtStreamWaitEvent(infinirtStream_t stream, infinirtEvent_t event) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
}

// ---- events --------------------------------------------------------------------------

__INFINI_C infiniStatus_t infinirtEventCreate(infinirtEvent_t *event_ptr) {
    RT_REQUIRE_PTR(event_ptr);
    RT_REQUIRE_NVIDIA();
    cudaEvent_t e = nullptr;
    cudaError_t err = cudaEventCreate(&e);
    *event_ptr = e;
    return fromCuda(err, "cudaEventCreate");
}

__INFINI_C infiniStatus_t infinirtEventCreateWithFlags(infinirtEvent_t *event_ptr, uint32_t flags) {
    RT_REQUIRE_PTR(event_ptr);
    RT_REQUIRE_NVIDIA();
    unsigned int cuda_flags = cudaEventDefault;
    if (flags & INFINIRT_EVENT_DISABLE_TIMING) {
        cuda_flags |= cudaEventDisableTiming;
    }
    if (flags & INFINIRT_EVENT_BLOCKING_SYNC) {
        cuda_flags |= cudaEventBlockingSync;
    }
    cudaEvent_t e = nullptr;
    cudaError_t err = cudaEventCreateWithFlags(&e, cuda_flags);
    *event_ptr = e;
    return fromCuda(err, "cudaEventCreateWithFlags");
}

__INFINI_C infiniStatus_t infinirtEventRecord(infinirtEvent_t event, infinirtStream_t stream) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
}

__INFINI_C infiniStatus_t infinirtEventQuery(infinirtEvent_t event, infinirtEventStatus_t *status_ptr) {
    RT_REQUIRE_PTR(status_ptr);
    RT_REQUIRE_NVIDIA();
    cudaError_t err = cudaEventQuery(static_cast<cudaEvent_t>(event));
    if (err == cudaSuccess) {
        *status_ptr = INFINIRT_EVENT_COMPLETE;
        return INFINI_STATUS_SUCCESS;
    }
    if (err == cudaErrorNotReady) {
        (void)cudaGetLastError();
        *status_ptr = INFINIRT_EVENT_NOT_READY;
        return INFINI_STATUS_SUCCESS;
    }
    return fromCuda(err, "cudaEventQuery");
}

__INFINI_C infiniStatus_t infinirtEventSynchronize(infinirtEvent_t event) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
}

__INFINI_C infiniStatus_t infinirtEventDestroy(infinirtEvent_t event) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
}

__INFINI_C infiniStatus_t infinirtEventElapsedTime(float *ms_ptr, infinirtEvent_t start, infinirtEvent_t end) {
    RT_REQUIRE_PTR(ms_ptr);
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaEventElapsedTime(ms_ptr, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(end)));
}

// ---- memory --------------------------------------------------------------------------

__INFINI_C infiniStatus_t infinirtMalloc(void **p_ptr, size_t size) {
    RT_REQUIRE_PTR(p_ptr);
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaMalloc(p_ptr, size));
}

__INFINI_C infiniStatus_t infinirtMallocHost(void **p_ptr, size_t size) {
    RT_REQUIRE_PTR(p_ptr);
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaMallocHost(p_ptr, size));
}

__INFINI_C infiniStatus_t infinirtFree(void *ptr) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaFree(ptr));
}

__INFINI_C infiniStatus_t infinirtFreeHost(void *ptr) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaFreeHost(ptr));
}

__INFINI_C infiniStatus_t infinirtMemcpy(void *dst, const void *src, size_t size, infinirtMemcpyKind_t kind) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaMemcpy(dst, src, size, toCudaKind(kind)));
}

__INFINI_C infiniStatus_t infinirtMemcpyAsync(void *dst, const void *src, size_t size, infinirtMemcpyKind_t kind, infinirtStream_t stream) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaMemcpyAsync(dst, src, size, toCudaKind(kind), static_cast<cudaStream_t>(stream)));
}

__INFINI_C infiniStatus_t infinirtMallocAsync(void **p_ptr, size_t size, infinirtStream_t stream) {
    RT_REQUIRE_PTR(p_ptr);
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaMallocAsync(p_ptr, size, static_cast<cudaStream_t>(stream)));
}

__INFINI_C infiniStatus_t infinirtFreeAsync(void *ptr, infinirtStream_t stream) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaFreeAsync(ptr, static_cast<cudaStream_t>(stream)));
}

__INFINI_C infiniStatus_t infinirtMemset(void *ptr, int value, size_t count) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaMemset(ptr, value, count));
}

__INFINI_C infiniStatus_t infinirtMemsetAsync(void *ptr, int value, size_t count, infinirtStream_t stream) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaMemsetAsync(ptr, value, count, static_cast<cudaStream_t>(stream)));
}

// ---- graph capture -------------------------------------------------------------------

__INFINI_C infiniStatus_t infinirtStreamBeginCapture(infinirtStream_t stream, infinirtStreamCaptureMode_t mode) {
    RT_REQUIRE_NVIDIA();
    cudaStreamCaptureMode cuda_mode = cudaStreamCaptureModeGlobal;
    if (mode == INFINIRT_STREAM_CAPTURE_MODE_THREAD_LOCAL) {
        cuda_mode = cudaStreamCaptureModeThreadLocal;
    } else if (mode == INFINIRT_STREAM_CAPTURE_MODE_RELAXED) {
        cuda_mode = cudaStreamCaptureModeRelaxed;
    }
    RT_CUDA(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cuda_mode));
}

__INFINI_C infiniStatus_t infinirtStreamEndCapture(infinirtStream_t stream, infinirtGraph_t *graph_ptr) {
    RT_REQUIRE_PTR(graph_ptr);
    RT_REQUIRE_NVIDIA();
    cudaGraph_t g = nullptr;
    cudaError_t err = cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &g);
    *graph_ptr = g;
    return fromCuda(err, "cudaStreamEndCapture");
}

__INFINI_C infiniStatus_t infinirtGraphDestroy(infinirtGraph_t graph) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaGraphDestroy(static_cast<cudaGraph_t>(graph)));
}

__INFINI_C infiniStatus_t infinirtGraphInstantiate(
    infinirtGraphExec_t *graph_exec_ptr,
    infinirtGraph_t graph,
    infinirtGraphNode_t *node_ptr,
    char *log_buffer,
    size_t buffer_size) {
    RT_REQUIRE_PTR(graph_exec_ptr);
    RT_REQUIRE_NVIDIA();
    (void)node_ptr;
    if (log_buffer != nullptr && buffer_size > 0) {
        log_buffer[0] = '\0';
    }
    cudaGraphExec_t exec = nullptr;
    cudaError_t err = cudaGraphInstantiate(&exec, static_cast<cudaGraph_t>(graph), 0);
    *graph_exec_ptr = exec;
    return fromCuda(err, "cudaGraphInstantiate");
}

__INFINI_C infiniStatus_t infinirtGraphExecDestroy(infinirtGraphExec_t graph_exec) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec)));
}

__INFINI_C infiniStatus_t infinirtGraphLuanch(infinirtGraphExec_t graph_exec, infinirtStream_t stream) {
    RT_REQUIRE_NVIDIA();
    RT_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), static_cast<cudaStream_t>(stream)));
}
