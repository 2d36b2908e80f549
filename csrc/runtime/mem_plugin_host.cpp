// Host side of the memory plugin ABI (csrc/abi/ogb_memory_abi.h): load a plugin, negotiate a version, read its vtable
// by the prefix rule, and expose allocate / free / stats / trim behind a plain C interface for the Python layer.
// Counterpart of the reference's allocator host loader (crates/onnx-runtime-memory-host/src/allocator.rs): a short or
// self-contradicting vtable is rejected at load, a slot above the effective level or absent is "unsupported", and no
// plugin failure propagates as anything but a status.
#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "abi/ogb_memory_abi.h"

namespace {

struct Plugin {
  void* lib = nullptr;
  OgbMemAllocator vt{};          // local copy: only the prefix the plugin filled in, the rest zero
  uint32_t level = 0;            // effective minor = min(declared, negotiated)
  decltype(&OgbMemDestroy) destroy = nullptr;
  std::mutex mu;
  uint64_t live = 0;
};

void set_err(char* err, int cap, const std::string& msg) {
  if (err && cap > 0) std::snprintf(err, static_cast<size_t>(cap), "%s", msg.c_str());
}

std::string describe(const OgbMemStatus& s) {
  char msg[sizeof(s.message) + 1];
  std::memcpy(msg, s.message, sizeof(s.message));
  msg[sizeof(s.message)] = 0;
  return "code " + std::to_string(s.code) + (msg[0] ? std::string(": ") + msg : std::string());
}

}  // namespace

extern "C" {

// Returns a handle or nullptr (with a message in err).  byte_limit 0 = no limit.
void* ogb_memhost_load(const char* path, uint64_t byte_limit, const char* purpose, char* err, int err_cap) {
  void* lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!lib) {
    set_err(err, err_cap, std::string("cannot load ") + path + ": " + dlerror());
    return nullptr;
  }
  auto negotiate = reinterpret_cast<decltype(&OgbMemNegotiate)>(dlsym(lib, "OgbMemNegotiate"));
  auto create = reinterpret_cast<decltype(&OgbMemCreate)>(dlsym(lib, "OgbMemCreate"));
  auto destroy = reinterpret_cast<decltype(&OgbMemDestroy)>(dlsym(lib, "OgbMemDestroy"));
  if (!negotiate || !create || !destroy) {
    set_err(err, err_cap, std::string(path) + " does not export OgbMemNegotiate, OgbMemCreate and OgbMemDestroy");
    dlclose(lib);
    return nullptr;
  }
  OgbMemVersion host{sizeof(OgbMemVersion), OGB_MEM_ABI_MAJOR, OGB_MEM_ABI_MINOR}, theirs{sizeof(OgbMemVersion), 0, 0};
  OgbMemStatus st = negotiate(&host, &theirs);
  if (st.code != OGB_MEM_OK || theirs.major != OGB_MEM_ABI_MAJOR) {
    set_err(err, err_cap, "version negotiation failed: host speaks " + std::to_string(OGB_MEM_ABI_MAJOR) + "." + std::to_string(OGB_MEM_ABI_MINOR) +
                              ", plugin answers " + std::to_string(theirs.major) + "." + std::to_string(theirs.minor) + " (" + describe(st) + ")");
    dlclose(lib);
    return nullptr;
  }
  const uint32_t negotiated = std::min<uint32_t>(theirs.minor, OGB_MEM_ABI_MINOR);
  OgbMemHostInfo info{sizeof(OgbMemHostInfo), negotiated, byte_limit, purpose};
  OgbMemAllocator filled;
  std::memset(&filled, 0, sizeof filled);
  filled.struct_size = sizeof filled;
  st = create(&info, &filled);
  if (st.code != OGB_MEM_OK) {
    set_err(err, err_cap, "the plugin could not create an allocator (" + describe(st) + ")");
    dlclose(lib);
    return nullptr;
  }
  // prefix rule: what the writer says it wrote, no more than we know about
  const size_t baseline = OGB_MEM_ALLOCATOR_BASELINE_SIZE;
  const size_t need = filled.abi_minor >= 1 ? sizeof(OgbMemAllocator) : baseline;
  if (filled.struct_size < baseline || filled.struct_size < need) {
    set_err(err, err_cap, "the plugin's vtable is " + std::to_string(filled.struct_size) + " bytes but it claims minor " +
                              std::to_string(filled.abi_minor) + ", which needs " + std::to_string(need) + ": it contradicts itself");
    destroy(&filled);
    dlclose(lib);
    return nullptr;
  }
  Plugin* p = new (std::nothrow) Plugin();
  if (!p) {
    destroy(&filled);
    dlclose(lib);
    set_err(err, err_cap, "out of memory");
    return nullptr;
  }
  std::memset(&p->vt, 0, sizeof p->vt);
  std::memcpy(&p->vt, &filled, std::min<size_t>(filled.struct_size, sizeof p->vt));
  p->level = std::min<uint32_t>(filled.abi_minor, negotiated);
  if (p->level < 1) { p->vt.stats = nullptr; p->vt.trim = nullptr; }        // never call a slot above the effective level
  if (!p->vt.allocate || !p->vt.deallocate) {
    set_err(err, err_cap, "the plugin's vtable lacks allocate or deallocate");
    destroy(&filled);
    dlclose(lib);
    delete p;
    return nullptr;
  }
  p->lib = lib;
  p->destroy = destroy;
  return p;
}

int ogb_memhost_level(void* h) { return h ? static_cast<int>(static_cast<Plugin*>(h)->level) : -1; }
const char* ogb_memhost_name(void* h) { return h && static_cast<Plugin*>(h)->vt.name ? static_cast<Plugin*>(h)->vt.name : ""; }

// 0 on success, else an OgbMemCode; message in err.
int ogb_memhost_alloc(void* h, uint64_t bytes, uint64_t alignment, void** out, char* err, int err_cap) {
  Plugin* p = static_cast<Plugin*>(h);
  if (!p || !out) return OGB_MEM_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(p->mu);
  *out = nullptr;
  OgbMemStatus st = p->vt.allocate(p->vt.self, bytes, alignment, out);
  if (st.code != OGB_MEM_OK) {
    set_err(err, err_cap, describe(st));
    return static_cast<int>(st.code);
  }
  if (!*out || (alignment && (reinterpret_cast<uintptr_t>(*out) & (alignment - 1)))) {
    set_err(err, err_cap, "the plugin reported success but returned a null or misaligned pointer");
    return OGB_MEM_INTERNAL;
  }
  p->live += 1;
  return 0;
}

int ogb_memhost_free(void* h, void* ptr, char* err, int err_cap) {
  Plugin* p = static_cast<Plugin*>(h);
  if (!p || !ptr) return OGB_MEM_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(p->mu);
  OgbMemStatus st = p->vt.deallocate(p->vt.self, ptr);
  if (st.code != OGB_MEM_OK) {
    set_err(err, err_cap, describe(st));
    return static_cast<int>(st.code);
  }
  if (p->live) p->live -= 1;
  return 0;
}

// out4: bytes_in_use, bytes_peak, allocations_live, allocations_total.  OGB_MEM_UNSUPPORTED when the plugin has no stats slot.
int ogb_memhost_stats(void* h, uint64_t* out4, char* err, int err_cap) {
  Plugin* p = static_cast<Plugin*>(h);
  if (!p || !out4) return OGB_MEM_INVALID_ARGUMENT;
  if (!p->vt.stats) {
    set_err(err, err_cap, "this plugin (level " + std::to_string(p->level) + ") has no stats capability");
    return OGB_MEM_UNSUPPORTED;
  }
  OgbMemStats s;
  std::memset(&s, 0, sizeof s);
  s.struct_size = sizeof s;
  OgbMemStatus st = p->vt.stats(p->vt.self, &s);
  if (st.code != OGB_MEM_OK) {
    set_err(err, err_cap, describe(st));
    return static_cast<int>(st.code);
  }
  out4[0] = s.bytes_in_use; out4[1] = s.bytes_peak; out4[2] = s.allocations_live; out4[3] = s.allocations_total;
  return 0;
}

int ogb_memhost_trim(void* h, uint64_t* released, char* err, int err_cap) {
  Plugin* p = static_cast<Plugin*>(h);
  if (!p || !released) return OGB_MEM_INVALID_ARGUMENT;
  if (!p->vt.trim) {
    set_err(err, err_cap, "this plugin has no trim capability");
    return OGB_MEM_UNSUPPORTED;
  }
  OgbMemStatus st = p->vt.trim(p->vt.self, released);
  if (st.code != OGB_MEM_OK) set_err(err, err_cap, describe(st));
  return static_cast<int>(st.code);
}

// Refuses (returns the live count) while allocations are outstanding.
int ogb_memhost_unload(void* h, char* err, int err_cap) {
  Plugin* p = static_cast<Plugin*>(h);
  if (!p) return 0;
  if (p->live) {
    set_err(err, err_cap, std::to_string(p->live) + " allocation(s) are still live; free them before unloading the plugin");
    return static_cast<int>(p->live);
  }
  OgbMemStatus st = p->destroy(&p->vt);
  if (st.code != OGB_MEM_OK) {
    set_err(err, err_cap, describe(st));
    return -static_cast<int>(st.code);
  }
  dlclose(p->lib);
  delete p;
  return 0;
}

}  // extern "C"
