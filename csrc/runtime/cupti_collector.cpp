// GPU activity collector over CUPTI's activity API: every kernel launch, memcpy and memset of the process with its
// device-side start / end timestamps, grid, block, shared memory and stream, gathered asynchronously by CUPTI and
// handed to the tracer, which lays them beside the engine's host spans on one Perfetto timeline.
//
// Same role as the reference's CUPTI tracer back end (crates/onnx-runtime-tracer/src/cupti.rs:1-60: activity buffers,
// kernel records joined to host spans by correlation id).  CUPTI is opened at run time (dlopen), so the runtime library
// carries no link-time dependency on it and a machine without CUPTI gets an error string, not a load failure.  Tests put
// a stand-in library in its place that plays the buffer protocol with synthetic records.
//
// Buffer protocol: CUPTI asks for an empty buffer (request callback), fills it with variable-size records and returns it
// (complete callback, on a CUPTI-owned thread); records are walked with cuptiActivityGetNextRecord.  The complete
// callback copies what the tracer needs into a mutex-guarded vector and frees the buffer; nothing of CUPTI's outlives it.
#include <cxxabi.h>
#include <dlfcn.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#if __has_include(<cupti.h>)
#include <cupti.h>
#define OGB_HAVE_CUPTI_HEADERS 1
#else
#define OGB_HAVE_CUPTI_HEADERS 0
#endif

extern "C" {

// One device-side activity.  kind: 0 kernel, 1 memcpy, 2 memset.  For copies `bytes` is the size and `detail` the CUPTI
// copy kind (1 host-to-device, 2 device-to-host, 8 device-to-device, 10 peer-to-peer); for kernels `detail` is registers
// per thread and `bytes` static + dynamic shared memory.  Times are CUPTI timestamps in nanoseconds (ogb_cupti_now()).
struct OgbGpuActivity {
    uint64_t start_ns, end_ns;
    uint64_t bytes;
    uint32_t kind, device, stream, correlation;
    int32_t grid[3], block[3];
    uint32_t detail, name_id;
};

int ogb_cupti_start(const char* library, int with_copies);
int ogb_cupti_stop(void);
int ogb_cupti_flush(void);
int ogb_cupti_drain(OgbGpuActivity* out, int capacity);
int ogb_cupti_pending(void);
const char* ogb_cupti_name(uint32_t name_id);
const char* ogb_cupti_last_error(void);
uint64_t ogb_cupti_now(void);
uint64_t ogb_cupti_dropped(void);
int ogb_cupti_headers(void);

}  // extern "C"

namespace {

std::mutex g_mu;
std::string g_error;
std::vector<OgbGpuActivity> g_records;
std::vector<std::string> g_names;
std::unordered_map<std::string, uint32_t> g_name_ids;
std::atomic<uint64_t> g_dropped{0};
bool g_running = false;
bool g_copies = false;
void* g_lib = nullptr;

int fail(const std::string& why) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_error = why;
    return -1;
}

uint32_t intern(const char* name) {            // g_mu held
    std::string key = name ? name : "(unnamed)";
    auto it = g_name_ids.find(key);            // keyed by the name as CUPTI gives it (mangled): demangle once per kernel
    if (it != g_name_ids.end()) return it->second;
    std::string shown = key;
    if (key.rfind("_Z", 0) == 0) {
        int status = 0;
        char* plain = abi::__cxa_demangle(key.c_str(), nullptr, nullptr, &status);
        if (status == 0 && plain) shown = plain;
        free(plain);
    }
    uint32_t id = static_cast<uint32_t>(g_names.size());
    g_names.push_back(std::move(shown));
    g_name_ids.emplace(std::move(key), id);
    return id;
}

#if OGB_HAVE_CUPTI_HEADERS

constexpr size_t kBufferBytes = 4u << 20;
constexpr size_t kBufferAlign = 8;             // CUPTI wants activity buffers 8-byte aligned
constexpr size_t kMaxHeld = 4u << 20;          // records kept for the tracer; beyond this the oldest half is discarded

struct Api {
    CUptiResult (*register_callbacks)(CUpti_BuffersCallbackRequestFunc, CUpti_BuffersCallbackCompleteFunc) = nullptr;
    CUptiResult (*enable)(CUpti_ActivityKind) = nullptr;
    CUptiResult (*disable)(CUpti_ActivityKind) = nullptr;
    CUptiResult (*flush_all)(uint32_t) = nullptr;
    CUptiResult (*next_record)(uint8_t*, size_t, CUpti_Activity**) = nullptr;
    CUptiResult (*dropped)(CUcontext, uint32_t, size_t*) = nullptr;
    CUptiResult (*timestamp)(uint64_t*) = nullptr;
    CUptiResult (*result_string)(CUptiResult, const char**) = nullptr;
} g_api;

std::string describe(CUptiResult r) {
    const char* s = nullptr;
    if (g_api.result_string && g_api.result_string(r, &s) == CUPTI_SUCCESS && s) return std::string(s);
    return "CUPTI error " + std::to_string(static_cast<int>(r));
}

void CUPTIAPI on_buffer_request(uint8_t** buffer, size_t* size, size_t* max_records) {
    void* p = nullptr;
    if (posix_memalign(&p, kBufferAlign, kBufferBytes) != 0) p = nullptr;
    *buffer = static_cast<uint8_t*>(p);
    *size = p ? kBufferBytes : 0;
    *max_records = 0;                           // as many as fit
}

void take(const CUpti_Activity* rec) {         // g_mu held
    OgbGpuActivity a{};
    switch (rec->kind) {
        case CUPTI_ACTIVITY_KIND_KERNEL:
        case CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL: {
            auto* k = reinterpret_cast<const CUpti_ActivityKernel9*>(rec);
            a.kind = 0;
            a.start_ns = k->start, a.end_ns = k->end;
            a.device = k->deviceId, a.stream = k->streamId, a.correlation = k->correlationId;
            a.grid[0] = k->gridX, a.grid[1] = k->gridY, a.grid[2] = k->gridZ;
            a.block[0] = k->blockX, a.block[1] = k->blockY, a.block[2] = k->blockZ;
            a.bytes = static_cast<uint64_t>(k->staticSharedMemory) + static_cast<uint64_t>(k->dynamicSharedMemory);
            a.detail = k->registersPerThread;
            a.name_id = intern(k->name);
            break;
        }
        case CUPTI_ACTIVITY_KIND_MEMCPY: {
            auto* m = reinterpret_cast<const CUpti_ActivityMemcpy6*>(rec);
            a.kind = 1;
            a.start_ns = m->start, a.end_ns = m->end;
            a.device = m->deviceId, a.stream = m->streamId, a.correlation = m->correlationId;
            a.bytes = m->bytes;
            a.detail = m->copyKind;
            a.name_id = intern("memcpy");
            break;
        }
        case CUPTI_ACTIVITY_KIND_MEMSET: {
            auto* m = reinterpret_cast<const CUpti_ActivityMemset4*>(rec);
            a.kind = 2;
            a.start_ns = m->start, a.end_ns = m->end;
            a.device = m->deviceId, a.stream = m->streamId, a.correlation = m->correlationId;
            a.bytes = m->bytes;
            a.name_id = intern("memset");
            break;
        }
        default:
            return;
    }
    if (g_records.size() >= kMaxHeld / sizeof(OgbGpuActivity)) {       // nobody drains: keep the recent half
        size_t half = g_records.size() / 2;
        g_dropped += half;
        g_records.erase(g_records.begin(), g_records.begin() + static_cast<long>(half));
    }
    g_records.push_back(a);
}

void CUPTIAPI on_buffer_complete(CUcontext ctx, uint32_t stream, uint8_t* buffer, size_t /*size*/, size_t valid) {
    if (buffer && valid > 0) {
        std::lock_guard<std::mutex> lk(g_mu);
        CUpti_Activity* rec = nullptr;
        while (g_api.next_record(buffer, valid, &rec) == CUPTI_SUCCESS && rec) take(rec);
    }
    size_t lost = 0;
    if (g_api.dropped && g_api.dropped(ctx, stream, &lost) == CUPTI_SUCCESS) g_dropped += lost;
    free(buffer);
}

template <typename F>
bool resolve(void* lib, const char* name, F& slot) {
    slot = reinterpret_cast<F>(dlsym(lib, name));
    return slot != nullptr;
}

#endif  // OGB_HAVE_CUPTI_HEADERS

}  // namespace

extern "C" {

int ogb_cupti_headers(void) { return OGB_HAVE_CUPTI_HEADERS; }

const char* ogb_cupti_last_error(void) {
    static thread_local std::string copy;
    std::lock_guard<std::mutex> lk(g_mu);
    copy = g_error;
    return copy.c_str();
}

uint64_t ogb_cupti_dropped(void) { return g_dropped.load(); }

int ogb_cupti_pending(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    return static_cast<int>(g_records.size());
}

const char* ogb_cupti_name(uint32_t id) {
    static thread_local std::string copy;
    std::lock_guard<std::mutex> lk(g_mu);
    copy = id < g_names.size() ? g_names[id] : std::string();
    return copy.c_str();
}

int ogb_cupti_drain(OgbGpuActivity* out, int capacity) {
    std::lock_guard<std::mutex> lk(g_mu);
    int n = static_cast<int>(std::min<size_t>(g_records.size(), capacity > 0 ? static_cast<size_t>(capacity) : 0));
    if (n > 0) {
        std::memcpy(out, g_records.data(), sizeof(OgbGpuActivity) * static_cast<size_t>(n));
        g_records.erase(g_records.begin(), g_records.begin() + n);
    }
    return n;
}

#if OGB_HAVE_CUPTI_HEADERS

int ogb_cupti_start(const char* library, int with_copies) {
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_running) return 0;
    }
    if (!g_lib) {
        const bool named = library && *library;              // a named library is the only candidate: no silent fallback
        const char* names[] = {named ? library : "libcupti.so.12", named ? nullptr : "libcupti.so"};
        std::string tried;
        for (const char* n : names) {
            if (!n) continue;
            g_lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
            if (g_lib) break;
            const char* e = dlerror();
            tried += std::string(tried.empty() ? "" : "; ") + n + ": " + (e ? e : "not found");
        }
        if (!g_lib) return fail("CUPTI library not found (" + tried + ")");
        bool ok = resolve(g_lib, "cuptiActivityRegisterCallbacks", g_api.register_callbacks) &
                  resolve(g_lib, "cuptiActivityEnable", g_api.enable) & resolve(g_lib, "cuptiActivityDisable", g_api.disable) &
                  resolve(g_lib, "cuptiActivityFlushAll", g_api.flush_all) &
                  resolve(g_lib, "cuptiActivityGetNextRecord", g_api.next_record) & resolve(g_lib, "cuptiGetTimestamp", g_api.timestamp);
        resolve(g_lib, "cuptiActivityGetNumDroppedRecords", g_api.dropped);          // optional
        resolve(g_lib, "cuptiGetResultString", g_api.result_string);                // optional
        if (!ok) {
            dlclose(g_lib);
            g_lib = nullptr;
            g_api = Api{};
            return fail("the CUPTI library lacks an activity entry point this collector needs");
        }
    }
    CUptiResult r = g_api.register_callbacks(on_buffer_request, on_buffer_complete);
    if (r != CUPTI_SUCCESS) return fail("cuptiActivityRegisterCallbacks: " + describe(r));
    r = g_api.enable(CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL);
    if (r != CUPTI_SUCCESS) return fail("cuptiActivityEnable(kernels): " + describe(r));
    if (with_copies) {
        CUptiResult a = g_api.enable(CUPTI_ACTIVITY_KIND_MEMCPY), b = g_api.enable(CUPTI_ACTIVITY_KIND_MEMSET);
        if (a != CUPTI_SUCCESS || b != CUPTI_SUCCESS) {
            g_api.disable(CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL);
            return fail("cuptiActivityEnable(copies): " + describe(a != CUPTI_SUCCESS ? a : b));
        }
    }
    std::lock_guard<std::mutex> lk(g_mu);
    g_running = true, g_copies = with_copies != 0;
    g_error.clear();
    return 0;
}

int ogb_cupti_flush(void) {
    if (!g_lib || !g_api.flush_all) return fail("the collector was never started");
    CUptiResult r = g_api.flush_all(1);        // 1: also hand back buffers that are not full yet
    if (r != CUPTI_SUCCESS) return fail("cuptiActivityFlushAll: " + describe(r));
    return 0;
}

int ogb_cupti_stop(void) {
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_running) return 0;
    }
    int rc = ogb_cupti_flush();
    g_api.disable(CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL);
    if (g_copies) {
        g_api.disable(CUPTI_ACTIVITY_KIND_MEMCPY);
        g_api.disable(CUPTI_ACTIVITY_KIND_MEMSET);
    }
    std::lock_guard<std::mutex> lk(g_mu);
    g_running = false;
    return rc;
}

uint64_t ogb_cupti_now(void) {
    uint64_t t = 0;
    if (g_api.timestamp) g_api.timestamp(&t);
    return t;
}

#else  // built on a machine without the CUPTI headers

int ogb_cupti_start(const char*, int) { return fail("built without the CUPTI headers: no GPU activity collector in this library"); }
int ogb_cupti_flush(void) { return fail("built without the CUPTI headers"); }
int ogb_cupti_stop(void) { return 0; }
uint64_t ogb_cupti_now(void) { return 0; }

#endif

}  // extern "C"
