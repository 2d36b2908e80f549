/* Example memory plugin: aligned host allocations with accounting and a byte limit.
 *
 * Build:  gcc -shared -fPIC -O2 -I csrc/abi examples/plugins/arena_allocator.c -o libarena_allocator.so
 *
 * Compile-time switches produce the misbehaving variants the host loader is tested against:
 *   -DPLUGIN_MINOR0        a plugin written to the baseline: shorter vtable, no stats / trim
 *   -DPLUGIN_MAJOR=2       a plugin of another major version: negotiation fails
 *   -DPLUGIN_LIES          claims minor 1 but hands over a baseline-sized vtable (contradicts itself)
 *   -DPLUGIN_FAIL_AFTER=n  the n-th allocation fails with OUT_OF_MEMORY
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ogb_memory_abi.h"

#ifndef PLUGIN_MAJOR
#define PLUGIN_MAJOR OGB_MEM_ABI_MAJOR
#endif

typedef struct Header {
  uint64_t bytes;
  void* base;
} Header;

typedef struct Arena {
  uint64_t limit, in_use, peak, live, total;
} Arena;

static OgbMemStatus status(uint32_t code, const char* msg) {
  OgbMemStatus s;
  memset(&s, 0, sizeof s);
  s.struct_size = sizeof s;
  s.code = code;
  if (msg) snprintf(s.message, sizeof s.message, "%s", msg);
  return s;
}

static OgbMemStatus arena_allocate(void* self, uint64_t bytes, uint64_t alignment, void** out_ptr) {
  Arena* a = (Arena*)self;
  if (!out_ptr || bytes == 0) return status(OGB_MEM_INVALID_ARGUMENT, "allocate needs a size and an out pointer");
  if (alignment < sizeof(void*)) alignment = sizeof(void*);
  if (alignment & (alignment - 1)) return status(OGB_MEM_INVALID_ARGUMENT, "alignment must be a power of two");
#ifdef PLUGIN_FAIL_AFTER
  if (a->total + 1 >= PLUGIN_FAIL_AFTER) return status(OGB_MEM_OUT_OF_MEMORY, "injected allocation failure");
#endif
  if (a->limit && a->in_use + bytes > a->limit) {
    char msg[120];
    snprintf(msg, sizeof msg, "%llu bytes requested, %llu of %llu in use", (unsigned long long)bytes, (unsigned long long)a->in_use,
             (unsigned long long)a->limit);
    return status(OGB_MEM_OUT_OF_MEMORY, msg);
  }
  void* base = malloc(bytes + alignment + sizeof(Header));
  if (!base) return status(OGB_MEM_OUT_OF_MEMORY, "malloc failed");
  uintptr_t p = ((uintptr_t)base + sizeof(Header) + alignment - 1) & ~(uintptr_t)(alignment - 1);
  Header* h = (Header*)(p - sizeof(Header));
  h->bytes = bytes;
  h->base = base;
  a->in_use += bytes;
  if (a->in_use > a->peak) a->peak = a->in_use;
  a->live += 1;
  a->total += 1;
  *out_ptr = (void*)p;
  return status(OGB_MEM_OK, NULL);
}

static OgbMemStatus arena_deallocate(void* self, void* ptr) {
  Arena* a = (Arena*)self;
  if (!ptr) return status(OGB_MEM_INVALID_ARGUMENT, "deallocate of NULL");
  Header* h = (Header*)((uintptr_t)ptr - sizeof(Header));
  a->in_use -= h->bytes;
  a->live -= 1;
  free(h->base);
  return status(OGB_MEM_OK, NULL);
}

#ifndef PLUGIN_MINOR0
static OgbMemStatus arena_stats(void* self, OgbMemStats* out) {
  Arena* a = (Arena*)self;
  if (!out || out->struct_size < sizeof(OgbMemStats)) return status(OGB_MEM_INVALID_ARGUMENT, "stats buffer too small");
  out->bytes_in_use = a->in_use;
  out->bytes_peak = a->peak;
  out->allocations_live = a->live;
  out->allocations_total = a->total;
  return status(OGB_MEM_OK, NULL);
}
#endif

OgbMemStatus OgbMemNegotiate(const OgbMemVersion* host, OgbMemVersion* plugin) {
  if (!host || !plugin || host->struct_size < sizeof(OgbMemVersion)) return status(OGB_MEM_INVALID_ARGUMENT, "bad version struct");
  plugin->struct_size = sizeof(OgbMemVersion);
  plugin->major = PLUGIN_MAJOR;
#ifdef PLUGIN_MINOR0
  plugin->minor = 0;
#else
  plugin->minor = host->minor < OGB_MEM_ABI_MINOR ? host->minor : OGB_MEM_ABI_MINOR;
#endif
  if (host->major != PLUGIN_MAJOR) return status(OGB_MEM_VERSION_MISMATCH, "this plugin speaks another major version");
  return status(OGB_MEM_OK, NULL);
}

OgbMemStatus OgbMemCreate(const OgbMemHostInfo* host, OgbMemAllocator* out) {
  if (!host || !out) return status(OGB_MEM_INVALID_ARGUMENT, "create needs host info and an out vtable");
  Arena* a = (Arena*)calloc(1, sizeof(Arena));
  if (!a) return status(OGB_MEM_OUT_OF_MEMORY, "no memory for the arena");
  a->limit = host->byte_limit;
  memset(out, 0, out->struct_size < sizeof(OgbMemAllocator) ? out->struct_size : sizeof(OgbMemAllocator));
  out->self = a;
  out->name = "arena";
  out->allocate = arena_allocate;
  out->deallocate = arena_deallocate;
#if defined(PLUGIN_MINOR0)
  out->struct_size = OGB_MEM_ALLOCATOR_BASELINE_SIZE;
  out->abi_minor = 0;
#elif defined(PLUGIN_LIES)
  out->struct_size = OGB_MEM_ALLOCATOR_BASELINE_SIZE;
  out->abi_minor = 1;
#else
  out->struct_size = sizeof(OgbMemAllocator);
  out->abi_minor = host->abi_minor < 1 ? host->abi_minor : 1;
  out->stats = arena_stats;
  out->trim = NULL; /* optional and absent: the host must report "unsupported", not succeed */
#endif
  return status(OGB_MEM_OK, NULL);
}

OgbMemStatus OgbMemDestroy(OgbMemAllocator* allocator) {
  if (!allocator || !allocator->self) return status(OGB_MEM_INVALID_ARGUMENT, "destroy of an empty allocator");
  Arena* a = (Arena*)allocator->self;
  if (a->live) return status(OGB_MEM_INVALID_ARGUMENT, "allocations are still live");
  free(a);
  allocator->self = NULL;
  return status(OGB_MEM_OK, NULL);
}
