/* Stand-in for libcupti in tests/test_gpu_activity_cpu.py: plays the activity-buffer protocol (request a buffer, fill it with
 * variable-size records, hand it back, walk it with cuptiActivityGetNextRecord) with a few synthetic records, using the real
 * header's record layouts.  FAKE_CUPTI_FAIL_ENABLE=1 makes cuptiActivityEnable refuse, as CUPTI does without privileges. */
#include <cupti.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

static CUpti_BuffersCallbackRequestFunc g_request;
static CUpti_BuffersCallbackCompleteFunc g_complete;
static int g_kernels, g_copies, g_sets, g_flushes;
static size_t g_dropped_once = 2;

static size_t aligned(size_t n) { return (n + 7) & ~(size_t)7; }

static size_t record_size(CUpti_ActivityKind kind) {
    switch (kind) {
        case CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL: return aligned(sizeof(CUpti_ActivityKernel9));
        case CUPTI_ACTIVITY_KIND_MEMCPY: return aligned(sizeof(CUpti_ActivityMemcpy6));
        case CUPTI_ACTIVITY_KIND_MEMSET: return aligned(sizeof(CUpti_ActivityMemset4));
        case CUPTI_ACTIVITY_KIND_DRIVER: return aligned(sizeof(CUpti_ActivityAPI));
        default: return 0;
    }
}

CUptiResult cuptiGetTimestamp(uint64_t* t) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    *t = (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
    return CUPTI_SUCCESS;
}

CUptiResult cuptiGetResultString(CUptiResult r, const char** s) {
    *s = r == CUPTI_ERROR_INSUFFICIENT_PRIVILEGES ? "CUPTI_ERROR_INSUFFICIENT_PRIVILEGES" : "CUPTI_ERROR";
    return CUPTI_SUCCESS;
}

CUptiResult cuptiActivityRegisterCallbacks(CUpti_BuffersCallbackRequestFunc req, CUpti_BuffersCallbackCompleteFunc done) {
    g_request = req, g_complete = done;
    return CUPTI_SUCCESS;
}

CUptiResult cuptiActivityEnable(CUpti_ActivityKind kind) {
    const char* f = getenv("FAKE_CUPTI_FAIL_ENABLE");
    if (f && *f == '1') return CUPTI_ERROR_INSUFFICIENT_PRIVILEGES;
    if (kind == CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL) g_kernels = 1;
    if (kind == CUPTI_ACTIVITY_KIND_MEMCPY) g_copies = 1;
    if (kind == CUPTI_ACTIVITY_KIND_MEMSET) g_sets = 1;
    return CUPTI_SUCCESS;
}

CUptiResult cuptiActivityDisable(CUpti_ActivityKind kind) {
    if (kind == CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL) g_kernels = 0;
    if (kind == CUPTI_ACTIVITY_KIND_MEMCPY) g_copies = 0;
    if (kind == CUPTI_ACTIVITY_KIND_MEMSET) g_sets = 0;
    return CUPTI_SUCCESS;
}

CUptiResult cuptiActivityGetNumDroppedRecords(CUcontext ctx, uint32_t stream, size_t* dropped) {
    (void)ctx, (void)stream;
    *dropped = g_dropped_once;
    g_dropped_once = 0;
    return CUPTI_SUCCESS;
}

CUptiResult cuptiActivityGetNextRecord(uint8_t* buffer, size_t valid, CUpti_Activity** record) {
    uint8_t* next = *record ? (uint8_t*)*record + record_size((*record)->kind) : buffer;
    if (next >= buffer + valid) {
        *record = NULL;
        return CUPTI_ERROR_MAX_LIMIT_REACHED;
    }
    *record = (CUpti_Activity*)next;
    return CUPTI_SUCCESS;
}

CUptiResult cuptiActivityFlushAll(uint32_t flag) {
    (void)flag;
    if (!g_request || !g_complete) return CUPTI_ERROR_NOT_INITIALIZED;
    uint8_t* buf = NULL;
    size_t size = 0, max_records = 0, used = 0;
    g_request(&buf, &size, &max_records);
    if (!buf) return CUPTI_ERROR_OUT_OF_MEMORY;
    uint64_t now;
    cuptiGetTimestamp(&now);
    uint64_t t = now - 1000000;                                /* the activity happened within the last millisecond */
    static const char* names[] = {"gemm_bf16_tcgen05_kernel", "paged_decode_kernel", "gemm_bf16_tcgen05_kernel"};
    if (g_kernels) {
        for (int i = 0; i < 3; ++i) {
            CUpti_ActivityKernel9* k = (CUpti_ActivityKernel9*)(buf + used);
            memset(k, 0, sizeof(*k));
            k->kind = CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL;
            k->start = t + (uint64_t)i * 100000, k->end = k->start + 40000 + (uint64_t)i * 10000;
            k->deviceId = 0, k->streamId = 7 + (uint32_t)(i == 1), k->correlationId = 100 + (uint32_t)i + 10 * (uint32_t)g_flushes;
            k->gridX = 148, k->gridY = 1, k->gridZ = 1, k->blockX = 192, k->blockY = 1, k->blockZ = 1;
            k->staticSharedMemory = 1024, k->dynamicSharedMemory = 200704, k->registersPerThread = 96;
            k->name = names[i];
            used += record_size(k->kind);
        }
        CUpti_ActivityAPI* api = (CUpti_ActivityAPI*)(buf + used);   /* a kind the collector did not ask for: must be skipped */
        memset(api, 0, sizeof(*api));
        api->kind = CUPTI_ACTIVITY_KIND_DRIVER;
        used += record_size(api->kind);
    }
    if (g_copies) {
        CUpti_ActivityMemcpy6* m = (CUpti_ActivityMemcpy6*)(buf + used);
        memset(m, 0, sizeof(*m));
        m->kind = CUPTI_ACTIVITY_KIND_MEMCPY;
        m->copyKind = CUPTI_ACTIVITY_MEMCPY_KIND_HTOD;
        m->bytes = 4096, m->start = t + 400000, m->end = m->start + 5000, m->streamId = 7, m->correlationId = 200;
        used += record_size(m->kind);
    }
    if (g_sets) {
        CUpti_ActivityMemset4* m = (CUpti_ActivityMemset4*)(buf + used);
        memset(m, 0, sizeof(*m));
        m->kind = CUPTI_ACTIVITY_KIND_MEMSET;
        m->bytes = 512, m->start = t + 500000, m->end = m->start + 2000, m->streamId = 7, m->correlationId = 201;
        used += record_size(m->kind);
    }
    ++g_flushes;
    g_complete(NULL, 0, buf, size, used);
    return CUPTI_SUCCESS;
}
