/*
 * Memory plugin ABI: a shared library that provides host allocations to the engine (pinned staging, swap space, the
 * host tier of the KV offload connector) without linking against it.  This header is the whole contract; a plugin may
 * be written in C.  Same principles as the reference's allocator ABI
 * (crates/onnx-runtime-memory-abi/include/nxmem_memory_abi.h): three exported symbols, every struct starts with its own
 * size, a major version that gates compatibility and a minor version that only appends fields, status codes instead of
 * exceptions, and a NULL optional slot that means "not supported", never "silently succeeds".
 *
 * Exported by a plugin:
 *   OgbMemNegotiate   agree on a version (the host proposes, the plugin answers what it implements)
 *   OgbMemCreate      fill an allocator vtable
 *   OgbMemDestroy     release the allocator (after every allocation has been freed)
 *
 * Reading rule for both sides: read struct_size first; copy min(struct_size, sizeof(local)) bytes into a zeroed local;
 * reject a struct smaller than the baseline of the minor version it claims; never call a slot that lies beyond the
 * copied prefix or above the negotiated minor.
 */
#ifndef OGB_MEMORY_ABI_H
#define OGB_MEMORY_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OGB_MEM_ABI_MAJOR 1u
#define OGB_MEM_ABI_MINOR 1u /* minor 1 appended `stats` and `trim` */

typedef enum OgbMemCode {
  OGB_MEM_OK = 0,
  OGB_MEM_OUT_OF_MEMORY = 1,
  OGB_MEM_INVALID_ARGUMENT = 2,
  OGB_MEM_UNSUPPORTED = 3,
  OGB_MEM_VERSION_MISMATCH = 4,
  OGB_MEM_INTERNAL = 5
} OgbMemCode;

typedef struct OgbMemStatus {
  uint32_t struct_size;
  uint32_t code;     /* OgbMemCode */
  char message[120]; /* NUL-terminated, may be empty */
} OgbMemStatus;

typedef struct OgbMemVersion {
  uint32_t struct_size;
  uint32_t major;
  uint32_t minor;
} OgbMemVersion;

typedef struct OgbMemStats {
  uint32_t struct_size;
  uint32_t reserved;
  uint64_t bytes_in_use;
  uint64_t bytes_peak;
  uint64_t allocations_live;
  uint64_t allocations_total;
} OgbMemStats;

/* What the host tells the plugin about itself. */
typedef struct OgbMemHostInfo {
  uint32_t struct_size;
  uint32_t abi_minor;       /* the negotiated minor */
  uint64_t byte_limit;      /* 0 = none; the plugin must fail allocations beyond it */
  const char* purpose;      /* e.g. "kv-swap", may be NULL */
} OgbMemHostInfo;

typedef struct OgbMemAllocator {
  uint32_t struct_size;
  uint32_t abi_minor;       /* the level this vtable implements (<= negotiated) */
  void* self;               /* passed back as the first argument of every slot */
  const char* name;         /* static string owned by the plugin */
  /* baseline (minor 0) */
  OgbMemStatus (*allocate)(void* self, uint64_t bytes, uint64_t alignment, void** out_ptr);
  OgbMemStatus (*deallocate)(void* self, void* ptr);
  /* minor 1, optional: NULL means unsupported */
  OgbMemStatus (*stats)(void* self, OgbMemStats* out);
  OgbMemStatus (*trim)(void* self, uint64_t* out_released_bytes);
} OgbMemAllocator;

#define OGB_MEM_ALLOCATOR_BASELINE_SIZE (offsetof(OgbMemAllocator, stats))

#if defined(_WIN32)
#define OGB_MEM_EXPORT __declspec(dllexport)
#else
#define OGB_MEM_EXPORT __attribute__((visibility("default")))
#endif

OGB_MEM_EXPORT OgbMemStatus OgbMemNegotiate(const OgbMemVersion* host, OgbMemVersion* plugin);
OGB_MEM_EXPORT OgbMemStatus OgbMemCreate(const OgbMemHostInfo* host, OgbMemAllocator* out);
OGB_MEM_EXPORT OgbMemStatus OgbMemDestroy(OgbMemAllocator* allocator);

#ifdef __cplusplus
}
#endif
#endif
