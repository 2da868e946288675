// Library state: error text, device/stream selection, storage entry points.
#include "common.cuh"

#include <atomic>
#include <cctype>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include <sched.h>

namespace ct {

namespace {
thread_local char g_err[512] = "";
std::mutex g_mutex;
DeviceState g_states[16];
std::atomic<int> g_device{-1};
std::atomic<cudaStream_t> g_stream{nullptr};
std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_precision{CT_PREC_3XTF32};
} // namespace

namespace {
std::recursive_mutex g_op_mutex;
}
OpLock::OpLock() { g_op_mutex.lock(); }
OpLock::~OpLock() { g_op_mutex.unlock(); }

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

ct_status fail(ct_status code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

ct_status cuda_fail(cudaError_t e, const char *what) {
    snprintf(g_err, sizeof(g_err), "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver)
        return CT_ERR_NO_DEVICE;
    return CT_ERR_CUDA;
}

cudaStream_t stream() { return g_stream.load(); }
void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Settings a host can give through the environment, read once, when the library is first used:
//   CAMEL_TENSOR_PRECISION = 3xtf32 | bf16   arithmetic of the tensor-core contractions
//   CAMEL_TENSOR_DEVICES   = "2" or "0,1,2,3" the GPU of this process: with a list, the entry at
//                            index LOCAL_RANK (else CAMEL_TENSOR_RANK, else 0) modulo its length -
//                            one process per GPU, each rank picking its own device from one setting
// ct_set_precision / ct_set_device override them.  A malformed value is an error, not a default.
ct_status settings_from_environment(int device_count, int *device_out) {
    if (const char *p = getenv("CAMEL_TENSOR_PRECISION")) {
        if (!strcmp(p, "3xtf32") || !strcmp(p, "3xTF32"))
            g_precision.store(CT_PREC_3XTF32);
        else if (!strcmp(p, "bf16") || !strcmp(p, "BF16"))
            g_precision.store(CT_PREC_BF16);
        else if (*p)
            return fail(CT_ERR_INVALID, "CAMEL_TENSOR_PRECISION=%s: expected 3xtf32 or bf16", p);
    }
    *device_out = -1;
    const char *d = getenv("CAMEL_TENSOR_DEVICES");
    if (!d || !*d)
        return CT_OK;
    std::vector<int> list;
    for (const char *c = d; *c;) {
        if (*c == ',' || *c == ' ') {
            ++c;
            continue;
        }
        char *end = nullptr;
        long v    = strtol(c, &end, 10);
        if (end == c || v < 0 || v >= device_count)
            return fail(CT_ERR_INVALID, "CAMEL_TENSOR_DEVICES=%s: expected device indices below %d", d, device_count);
        list.push_back((int)v);
        c = end;
    }
    if (list.empty())
        return CT_OK;
    long rank = 0;
    if (const char *r = getenv("LOCAL_RANK"))
        rank = strtol(r, nullptr, 10);
    else if (const char *r2 = getenv("CAMEL_TENSOR_RANK"))
        rank = strtol(r2, nullptr, 10);
    if (rank < 0)
        rank = 0;
    *device_out = list[(size_t)rank % list.size()];
    return CT_OK;
}

ct_status current(DeviceState **out) {
    int dev = g_device.load();
    if (dev < 0) {
        std::lock_guard<std::mutex> lock(g_mutex);
        dev = g_device.load();
        if (dev < 0) {
            int count     = 0;
            cudaError_t e = cudaGetDeviceCount(&count);
            if (e != cudaSuccess || count == 0) {
                cudaGetLastError();
                return fail(CT_ERR_NO_DEVICE, "no CUDA device: libcamel_tensor_b200 has no CPU fallback");
            }
            int chosen = -1;
            CT_TRY(settings_from_environment(count, &chosen));
            if (chosen >= 0)
                CT_CUDA(cudaSetDevice(chosen));
            CT_CUDA(cudaGetDevice(&dev));
            g_device.store(dev);
        }
    }
    if (dev >= 16)
        return fail(CT_ERR_INVALID, "device index %d not supported", dev);
    // The selected device is a property of the process (ct_set_device), the CUDA "current device"
    // one of the calling thread: a scheduler's worker threads start on device 0 whatever another
    // thread selected.  Every entry point passes through here, so the thread is moved first.
    int thread_dev = -1;
    CT_CUDA(cudaGetDevice(&thread_dev));
    if (thread_dev != dev)
        CT_CUDA(cudaSetDevice(dev));
    DeviceState *st = &g_states[dev];
    if (!st->ready) {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!st->ready) {
            CT_CUDA(cudaSetDevice(dev));
            cudaDeviceProp prop;
            CT_CUDA(cudaGetDeviceProperties(&prop, dev));
            if (prop.major != 10)
                return fail(
                    CT_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                    dev, prop.major, prop.minor);
            st->device   = dev;
            st->sm_count = prop.multiProcessorCount;
            CT_CUDA(cudaMalloc(&st->flags_dev, FLAG_COUNT * sizeof(uint32_t)));
            CT_CUDA(cudaMemset(st->flags_dev, 0, FLAG_COUNT * sizeof(uint32_t)));
            CT_CUDA(cudaMallocHost(&st->flags_host, FLAG_COUNT * sizeof(uint32_t)));
            memset(st->flags_host, 0, FLAG_COUNT * sizeof(uint32_t));
            // Tensor storage comes from the device's stream-ordered pool; keep freed blocks cached
            // instead of returning them to the driver at every synchronisation.
            cudaMemPool_t pool;
            CT_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
            uint64_t keep = UINT64_MAX;
            CT_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
            st->ready = true;
        }
    }
    *out = st;
    return CT_OK;
}

ct_status ensure_ws(void **ptr, size_t *cap, size_t bytes) {
    if (*cap >= bytes && *ptr)
        return CT_OK;
    // growing means cudaFree + cudaMalloc, which a stream that is being recorded cannot do
    cudaStreamCaptureStatus cap_state = cudaStreamCaptureStatusNone;
    CT_CUDA(cudaStreamIsCapturing(stream(), &cap_state));
    if (cap_state != cudaStreamCaptureStatusNone)
        return fail(
            CT_ERR_INVALID,
            "a workspace would have to grow to %zu bytes while calls are being recorded: run the sequence once "
            "before ct_graph_begin",
            bytes);
    if (*ptr) {
        CT_CUDA(cudaStreamSynchronize(stream()));
        CT_CUDA(cudaFree(*ptr));
        *ptr = nullptr;
        *cap = 0;
    }
    size_t want = bytes + bytes / 8 + 256;
    CT_CUDA(cudaMalloc(ptr, want));
    *cap = want;
    return CT_OK;
}

ct_status clear_data_flags(DeviceState *st) {
    static_assert(FLAG_DIV_ZERO == 0 && FLAG_LOG_DOMAIN == 1 && FLAG_TIMEOUT == 2, "layout of the error words");
    CT_CUDA(cudaMemsetAsync(st->flags_dev, 0, 2 * sizeof(uint32_t), stream()));
    return CT_OK;
}

ct_status report_timeout(DeviceState *st, const char *what) {
    if (!st->flags_host[FLAG_TIMEOUT])
        return CT_OK;
    uint32_t where = st->flags_host[FLAG_TIMEOUT] - 1;
    CT_CUDA(cudaMemsetAsync(st->flags_dev + FLAG_TIMEOUT, 0, sizeof(uint32_t), stream()));
    return fail(
        CT_ERR_TIMEOUT,
        "%s: a bounded wait inside a contraction kernel ran out (block %u); outputs of contractions enqueued "
        "since then are undefined",
        what, where);
}

ct_status fetch_flags(DeviceState *st) {
    CT_CUDA(cudaMemcpyAsync(
        st->flags_host, st->flags_dev, FLAG_COUNT * sizeof(uint32_t), cudaMemcpyDeviceToHost,
        stream()));
    CT_CUDA(cudaStreamSynchronize(stream()));
    return CT_OK;
}

} // namespace ct

namespace ct {
namespace {
// CPUs local to a GPU, from /sys/bus/pci/devices/<bus id>/local_cpulist ("0-31,64-95").
bool local_cpus_of_device(int dev, cpu_set_t *set) {
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, (int)sizeof(bus), dev) != cudaSuccess)
        return false;
    for (char *c = bus; *c; ++c)
        *c = (char)tolower((unsigned char)*c);
    char path[128];
    snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/local_cpulist", bus);
    FILE *f = fopen(path, "r");
    if (!f)
        return false;
    char line[4096] = {0};
    bool got        = fgets(line, sizeof(line), f) != nullptr;
    fclose(f);
    if (!got)
        return false;
    CPU_ZERO(set);
    int count = 0;
    for (char *p = line; *p;) {
        if (!isdigit((unsigned char)*p)) {
            ++p;
            continue;
        }
        long a = strtol(p, &p, 10), b = a;
        if (*p == '-')
            b = strtol(p + 1, &p, 10);
        for (long c = a; c <= b && c < CPU_SETSIZE; ++c) {
            CPU_SET((int)c, set);
            ++count;
        }
    }
    return count > 0;
}
} // namespace
} // namespace ct


// ---- large copies from pageable host memory -------------------------------------------------
//
// The reference keeps tensors in ordinary (pageable) host memory, so that is what a program hands
// the module at a graph boundary.  cudaMemcpy from pageable memory is staged by the driver through
// its own buffers by one thread: measured 18 GB/s for 16 MB falling to 11 GB/s for 256 MB, against
// the 54 GB/s the link gives page-locked memory.  For sources of 32 MiB and more ct_h2d stages the
// copy itself: a few host threads copy chunks into a ring of page-locked buffers while earlier
// chunks are already on their way to the device (measured 28-32 GB/s at 64 MB, 28-40 GB/s at
// 256 MB).  Chunks are finished in order (workers claim consecutive chunks from one counter); the
// calling thread copies the first chunk (it is awake; the workers sleep between calls), then only
// issues transfers.  The hand-offs are atomics, not locks.  Below 32 MiB the plain path stays:
// waking the workers costs as much as they save.
namespace ct {
namespace {

#ifndef CT_STAGE_CHUNK_KB
#define CT_STAGE_CHUNK_KB 1024
#endif
#ifndef CT_STAGE_WORKERS
#define CT_STAGE_WORKERS 4
#endif
constexpr size_t kStageChunk   = (size_t)CT_STAGE_CHUNK_KB << 10;
constexpr size_t kStageRing    = 16u << 20;                   // page-locked bytes held by the ring
constexpr int kStageSlots      = (int)(kStageRing / kStageChunk);
constexpr int kStageWorkers    = CT_STAGE_WORKERS;
constexpr size_t kStageMinimum = 32u << 20; // smaller copies go the plain way: waking the workers costs more
                                            // than they save (12 MB: 650-1000 us staged, 690 us plain)

inline void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#else
    std::this_thread::yield();
#endif
}

class HostStager {
  public:
    // Copies `bytes` from pageable `src` to device `dst` on `s`.  On return every chunk has been
    // copied out of `src` and handed to the stream.
    cudaError_t copy(void *dst, const void *src, size_t bytes, cudaStream_t s) {
        std::lock_guard<std::mutex> whole(call_mutex_); // one staged copy at a time: the ring is shared
        cudaError_t e = ensure();
        if (e != cudaSuccess)
            return e;
        // transfers of an earlier call that the caller did not wait for still own their slots
        for (int i = 0; i < kStageSlots; ++i)
            if (slot_pending_[i]) {
                e = cudaEventSynchronize(slot_done_[i]);
                if (e != cudaSuccess)
                    return e;
                slot_pending_[i] = false;
            }
        src_    = static_cast<const char *>(src);
        bytes_  = bytes;
        chunks_ = (bytes + kStageChunk - 1) / kStageChunk;
        next_.store(1, std::memory_order_relaxed); // chunk 0 is this thread's
        retired_.store(0, std::memory_order_relaxed);
        abort_.store(false, std::memory_order_relaxed);
        {
            std::lock_guard<std::mutex> lock(mutex_);
            open_ = true;
            ++epoch_;
        }
        if (chunks_ > 1)
            wake_.notify_all();
        fill(0);

        size_t issued = 0, retired = 0;
        cudaError_t result = cudaSuccess;
        while (issued < chunks_) {
            const int slot = (int)(issued % kStageSlots);
            if (ready_[slot].load(std::memory_order_acquire) == base_ + issued + 1) {
                const size_t off = issued * kStageChunk;
                const size_t len = bytes - off < kStageChunk ? bytes - off : kStageChunk;
                e = cudaMemcpyAsync(static_cast<char *>(dst) + off, slot_mem_[slot], len, cudaMemcpyHostToDevice, s);
                if (e == cudaSuccess)
                    e = cudaEventRecord(slot_done_[slot], s);
                if (e != cudaSuccess) {
                    result = e;
                    break;
                }
                slot_pending_[slot] = true;
                ++issued;
            } else {
                cpu_relax();
            }
            // slots whose transfer has finished go back to the workers (only a copy longer than the
            // ring ever waits for one)
            if (chunks_ > (size_t)kStageSlots)
                while (retired < issued) {
                    cudaError_t q = cudaEventQuery(slot_done_[retired % kStageSlots]);
                    if (q == cudaErrorNotReady) {
                        cudaGetLastError();
                        break;
                    }
                    if (q != cudaSuccess) {
                        result = q;
                        break;
                    }
                    slot_pending_[retired % kStageSlots] = false;
                    ++retired;
                    retired_.store(retired, std::memory_order_release);
                }
            if (result != cudaSuccess)
                break;
        }
        // close the call: no worker may touch its state after this returns
        abort_.store(result != cudaSuccess, std::memory_order_release);
        next_.store(chunks_, std::memory_order_release);
        {
            std::lock_guard<std::mutex> lock(mutex_);
            open_ = false;
        }
        while (active_.load(std::memory_order_acquire) != 0)
            cpu_relax();
        base_ += chunks_; // chunk sequence numbers never repeat, so a stale mark cannot be mistaken
        return result;
    }

    ~HostStager() {
        {
            std::lock_guard<std::mutex> lock(mutex_);
            stop_ = true;
        }
        wake_.notify_all();
        for (auto &t : workers_)
            if (t.joinable())
                t.join();
    }

  private:
    cudaError_t ensure() {
        if (ready_state_)
            return cudaSuccess;
        for (int i = 0; i < kStageSlots; ++i) {
            cudaError_t e = cudaHostAlloc(&slot_mem_[i], kStageChunk, cudaHostAllocDefault);
            if (e == cudaSuccess)
                e = cudaEventCreateWithFlags(&slot_done_[i], cudaEventDisableTiming);
            if (e != cudaSuccess)
                return e;
            slot_pending_[i] = false;
            ready_[i].store(0, std::memory_order_relaxed);
        }
        for (int i = 0; i < kStageWorkers; ++i)
            workers_.emplace_back([this] { work(); });
        ready_state_ = true;
        return cudaSuccess;
    }

    // host copy of chunk c into its slot, once the slot's previous transfer is over
    void fill(size_t c) {
        while (c >= retired_.load(std::memory_order_acquire) + (size_t)kStageSlots) {
            if (abort_.load(std::memory_order_acquire))
                return;
            cpu_relax();
        }
        const int slot   = (int)(c % kStageSlots);
        const size_t off = c * kStageChunk;
        const size_t len = bytes_ - off < kStageChunk ? bytes_ - off : kStageChunk;
        memcpy(slot_mem_[slot], src_ + off, len);
        ready_[slot].store(base_ + c + 1, std::memory_order_release);
    }

    void work() {
        size_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lock(mutex_);
                wake_.wait(lock, [&] { return stop_ || (open_ && epoch_ != seen); });
                if (stop_)
                    return;
                seen = epoch_;
                active_.fetch_add(1, std::memory_order_acq_rel); // under the lock: copy() closes the call under it
            }
            for (;;) {
                const size_t c = next_.fetch_add(1, std::memory_order_acq_rel);
                if (c >= chunks_ || abort_.load(std::memory_order_acquire))
                    break;
                fill(c);
            }
            active_.fetch_sub(1, std::memory_order_acq_rel);
        }
    }

    std::mutex call_mutex_, mutex_;
    std::condition_variable wake_;
    std::vector<std::thread> workers_;
    void *slot_mem_[kStageSlots]        = {};
    cudaEvent_t slot_done_[kStageSlots] = {};
    bool slot_pending_[kStageSlots]     = {};
    std::atomic<size_t> ready_[kStageSlots];
    std::atomic<size_t> next_{0}, retired_{0};
    std::atomic<int> active_{0};
    std::atomic<bool> abort_{false};
    const char *src_ = nullptr;
    size_t bytes_ = 0, chunks_ = 0, base_ = 0, epoch_ = 0;
    bool ready_state_ = false, stop_ = false, open_ = false;
};

HostStager g_stager;

// true when `p` is ordinary host memory (not page-locked, not registered, not managed)
bool is_pageable(const void *p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return true;
    }
    return attr.type == cudaMemoryTypeUnregistered;
}

} // namespace
} // namespace ct

using namespace ct;

extern "C" {

const char *ct_last_error(void) { return g_err; }
const char *ct_version(void) { return "camel_tensor_b200 0.1 (sm_100a)"; }

ct_status ct_device_count(int *count_host) {
    if (!count_host)
        return fail(CT_ERR_INVALID, "count_host is null");
    int count     = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) {
        cudaGetLastError();
        count = 0;
    }
    *count_host = count;
    return CT_OK;
}

ct_status ct_set_device(int device) {
    int count     = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(CT_ERR_NO_DEVICE, "no CUDA device: libcamel_tensor_b200 has no CPU fallback");
    }
    if (device < 0 || device >= count)
        return fail(CT_ERR_INVALID, "device %d out of range (have %d)", device, count);
    CT_CUDA(cudaSetDevice(device));
    g_device.store(device);
    DeviceState *st;
    return current(&st);
}

ct_status ct_get_device(int *device_host) {
    if (!device_host)
        return fail(CT_ERR_INVALID, "device_host is null");
    DeviceState *st;
    CT_TRY(current(&st));
    *device_host = st->device;
    return CT_OK;
}

ct_status ct_set_stream(void *s) {
    g_stream.store(static_cast<cudaStream_t>(s));
    return CT_OK;
}

ct_status ct_sync(void) {
    DeviceState *st;
    CT_TRY(current(&st));
    CT_CUDA(cudaStreamSynchronize(stream()));
    return CT_OK;
}

uint64_t ct_launch_count(void) { return g_launches.load(); }

ct_status ct_set_precision(ct_precision p) {
    if (p != CT_PREC_3XTF32 && p != CT_PREC_BF16)
        return fail(CT_ERR_INVALID, "unknown precision %d", (int)p);
    g_precision.store((int)p);
    return CT_OK;
}

ct_precision ct_get_precision(void) { return (ct_precision)g_precision.load(); }

ct_status ct_alloc(void **ptr_dev, size_t bytes) {
    if (!ptr_dev)
        return fail(CT_ERR_INVALID, "ptr_dev is null");
    DeviceState *st;
    CT_TRY(current(&st));
    *ptr_dev = nullptr;
    if (bytes == 0)
        bytes = 1; // an empty tensor still owns a distinct address
    // stream-ordered, pooled: an operator result costs microseconds, not a device-wide stall
    CT_CUDA(cudaMallocAsync(ptr_dev, bytes, stream()));
    return CT_OK;
}

ct_status ct_free(void *ptr_dev) {
    if (!ptr_dev)
        return CT_OK;
    DeviceState *st;
    CT_TRY(current(&st));
    CT_CUDA(cudaFreeAsync(ptr_dev, stream()));
    return CT_OK;
}

ct_status ct_h2d(void *dst_dev, const void *src_host, size_t bytes) {
    DeviceState *st;
    CT_TRY(current(&st));
    if (bytes == 0)
        return CT_OK;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (bytes >= kStageMinimum && cudaStreamIsCapturing(stream(), &cap) == cudaSuccess &&
        cap == cudaStreamCaptureStatusNone && is_pageable(src_host)) {
        // a large pageable source: staged through page-locked chunks by several host threads
        CT_CUDA(g_stager.copy(dst_dev, src_host, bytes, stream()));
        CT_CUDA(cudaStreamSynchronize(stream()));
        return CT_OK;
    }
    CT_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, stream()));
    CT_CUDA(cudaStreamSynchronize(stream())); // src_host may be pageable and reused at once
    return CT_OK;
}

ct_status ct_d2h(void *dst_host, const void *src_dev, size_t bytes) {
    DeviceState *st;
    CT_TRY(current(&st));
    if (bytes == 0)
        return CT_OK;
    CT_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, stream()));
    CT_CUDA(cudaStreamSynchronize(stream()));
    return CT_OK;
}

// The host read at a graph boundary: the data and the device's error record in one trip (two
// copies enqueued, one synchronisation), then the error record reported as ct_check does.
ct_status ct_d2h_checked(void *dst_host, const void *src_dev, size_t bytes) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (bytes > 0)
        CT_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, stream()));
    CT_TRY(fetch_flags(st)); // synchronises the stream: both copies have landed
    return report_timeout(st, "ct_d2h_checked");
}

ct_status ct_d2d(void *dst_dev, const void *src_dev, size_t bytes) {
    DeviceState *st;
    CT_TRY(current(&st));
    if (bytes == 0)
        return CT_OK;
    CT_CUDA(cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice, stream()));
    return CT_OK;
}

ct_status ct_host_alloc(void **ptr_host, size_t bytes) {
    if (!ptr_host)
        return fail(CT_ERR_INVALID, "ptr_host is null");
    DeviceState *st;
    CT_TRY(current(&st));
    *ptr_host = nullptr;
    if (bytes == 0)
        return CT_OK;
    // Page-locked pages land on the memory node of the CPU that allocates them.  On a two-socket host
    // a buffer on the far socket crosses the inter-socket link on every copy and several GPUs then
    // share that link; so the calling thread is moved, for the duration of the allocation, onto the
    // CPUs that are local to the current GPU (as sysfs reports them), where the process is allowed there.
    cpu_set_t saved, local;
    bool moved = false;
    int dev    = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && sched_getaffinity(0, sizeof(saved), &saved) == 0 &&
        local_cpus_of_device(dev, &local)) {
        cpu_set_t both;
        CPU_AND(&both, &saved, &local);
        if (CPU_COUNT(&both) > 0 && !CPU_EQUAL(&both, &saved))
            moved = sched_setaffinity(0, sizeof(both), &both) == 0;
    }
    cudaError_t e = cudaHostAlloc(ptr_host, bytes, cudaHostAllocDefault);
    if (moved)
        sched_setaffinity(0, sizeof(saved), &saved);
    if (e != cudaSuccess)
        return cuda_fail(e, "cudaHostAlloc");
    return CT_OK;
}

ct_status ct_host_free(void *ptr_host) {
    if (!ptr_host)
        return CT_OK;
    CT_CUDA(cudaFreeHost(ptr_host));
    return CT_OK;
}

ct_status ct_h2d_async(void *dst_dev, const void *src_host_pinned, size_t bytes) {
    DeviceState *st;
    CT_TRY(current(&st));
    if (bytes == 0)
        return CT_OK;
    CT_CUDA(cudaMemcpyAsync(dst_dev, src_host_pinned, bytes, cudaMemcpyHostToDevice, stream()));
    return CT_OK;
}

ct_status ct_d2h_async(void *dst_host_pinned, const void *src_dev, size_t bytes) {
    DeviceState *st;
    CT_TRY(current(&st));
    if (bytes == 0)
        return CT_OK;
    CT_CUDA(cudaMemcpyAsync(dst_host_pinned, src_dev, bytes, cudaMemcpyDeviceToHost, stream()));
    return CT_OK;
}

ct_status ct_stream_create(void **stream_out) {
    if (!stream_out)
        return fail(CT_ERR_INVALID, "stream_out is null");
    DeviceState *st;
    CT_TRY(current(&st));
    cudaStream_t s = nullptr;
    CT_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream_out = s;
    return CT_OK;
}

ct_status ct_stream_destroy(void *s) {
    if (!s)
        return CT_OK;
    if (stream() == static_cast<cudaStream_t>(s))
        return fail(CT_ERR_INVALID, "ct_stream_destroy: the stream is the current one");
    CT_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(s)));
    return CT_OK;
}

ct_status ct_event_create(void **event_out) {
    if (!event_out)
        return fail(CT_ERR_INVALID, "event_out is null");
    DeviceState *st;
    CT_TRY(current(&st));
    cudaEvent_t e = nullptr;
    CT_CUDA(cudaEventCreate(&e));
    *event_out = e;
    return CT_OK;
}

ct_status ct_event_destroy(void *event) {
    if (!event)
        return CT_OK;
    CT_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
    return CT_OK;
}

ct_status ct_event_record(void *event) {
    if (!event)
        return fail(CT_ERR_INVALID, "event is null");
    CT_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), stream()));
    return CT_OK;
}

ct_status ct_stream_wait_event(void *event) {
    if (!event)
        return fail(CT_ERR_INVALID, "event is null");
    CT_CUDA(cudaStreamWaitEvent(stream(), static_cast<cudaEvent_t>(event), 0));
    return CT_OK;
}

ct_status ct_event_sync(void *event) {
    if (!event)
        return fail(CT_ERR_INVALID, "event is null");
    CT_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
    return CT_OK;
}

ct_status ct_event_elapsed_ms(void *start_event, void *end_event, float *ms_out) {
    if (!start_event || !end_event || !ms_out)
        return fail(CT_ERR_INVALID, "ct_event_elapsed_ms: null argument");
    CT_CUDA(cudaEventElapsedTime(ms_out, static_cast<cudaEvent_t>(start_event), static_cast<cudaEvent_t>(end_event)));
    return CT_OK;
}

ct_dtype ct_result_dtype(ct_binary_op op, ct_dtype lhs, ct_dtype rhs) {
    if (op == CT_DIV || op == CT_POW)
        return CT_F32;
    if (lhs == CT_F32 || rhs == CT_F32)
        return CT_F32;
    if (lhs == CT_I64 || rhs == CT_I64)
        return CT_I64;
    return CT_BOOL;
}

} // extern "C"

extern "C" ct_status ct_check(void) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    CT_TRY(fetch_flags(st));
    return report_timeout(st, "ct_check");
}

// Host-side fault injection for tests of the error path: writes one of the device error words in
// stream order, as if a kernel had raised it.  Nothing on the GPU waits, traps or faults.
extern "C" ct_status ct_inject_status(int word, uint32_t value) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (word < 0 || word >= FLAG_COUNT)
        return fail(CT_ERR_INVALID, "ct_inject_status: word %d out of range", word);
    // the value travels inside the memset, so the call needs no host buffer that outlives it
    if (value > 0xff)
        return fail(CT_ERR_INVALID, "ct_inject_status: value must fit one byte");
    CT_CUDA(cudaMemsetAsync(st->flags_dev + word, 0, sizeof(uint32_t), stream()));
    CT_CUDA(cudaMemsetAsync(st->flags_dev + word, (int)value, 1, stream()));
    return CT_OK;
}

// ---- per-kernel device timing -------------------------------------------------------------

namespace ct {
namespace {
struct ProfRecord {
    const char *name;
    cudaEvent_t e0, e1;
};
std::atomic<int> g_prof_on{0};
std::mutex g_prof_mutex;
std::vector<ProfRecord> g_prof;
} // namespace

bool profiling_enabled() { return g_prof_on.load(std::memory_order_relaxed) != 0; }

ProfScope::ProfScope(const char *name) : name_(name), e0_(nullptr), e1_(nullptr) {
    if (!g_prof_on.load(std::memory_order_relaxed))
        return;
    if (cudaEventCreate(&e0_) != cudaSuccess || cudaEventCreate(&e1_) != cudaSuccess) {
        e0_ = e1_ = nullptr;
        return;
    }
    cudaEventRecord(e0_, stream());
}

ProfScope::~ProfScope() {
    if (!e0_)
        return;
    cudaEventRecord(e1_, stream());
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof.push_back(ProfRecord{name_, e0_, e1_});
}
} // namespace ct

extern "C" ct_status ct_profile_enable(int on) {
    g_prof_on.store(on ? 1 : 0);
    return CT_OK;
}

extern "C" ct_status ct_profile_read(const char *kernel, double *total_ms_host, uint64_t *launches_host) {
    DeviceState *st;
    CT_TRY(current(&st));
    CT_CUDA(cudaStreamSynchronize(stream()));
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    double total = 0.0;
    uint64_t count = 0;
    std::vector<ProfRecord> keep;
    for (auto &r : g_prof) {
        if (kernel && strcmp(kernel, r.name) != 0) {
            keep.push_back(r);
            continue;
        }
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess) {
            total += ms;
            ++count;
        }
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    g_prof.swap(keep);
    if (total_ms_host)
        *total_ms_host = total;
    if (launches_host)
        *launches_host = count;
    return CT_OK;
}
