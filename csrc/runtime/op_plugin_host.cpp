// Host side of the operator plugin ABI (csrc/abi/ogb_kernel_abi.h): load a plugin, negotiate version and capabilities,
// read its provider by the prefix rule, list its kernels, and run them behind a plain C interface for the Python layer.
// Counterpart of the reference's native EP plugin host (crates/onnx-runtime-ep-nxrt-abi/src/version.rs
// `validate_negotiation`, vtable.rs): a wrong major, an unknown capability bit, a short or incomplete vtable are refusals
// at load; a kernel's failure is a status with the plugin's message, never an exception across the boundary.
#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "abi/ogb_kernel_abi.h"

namespace {

struct OpPlugin {
  void* lib = nullptr;
  OgbOpProvider vt{};
  uint32_t capabilities = 0;
  std::vector<OgbOpKernelDesc> kernels;
  int live_kernels = 0;
};

struct OpKernel {
  OpPlugin* owner = nullptr;
  OgbOpKernel vt{};
};

void set_err(char* err, int cap, const std::string& msg) {
  if (err && cap > 0) std::snprintf(err, static_cast<size_t>(cap), "%s", msg.c_str());
}

std::string describe(const OgbOpStatus& s) {
  char msg[sizeof(s.message) + 1];
  std::memcpy(msg, s.message, sizeof(s.message));
  msg[sizeof(s.message)] = 0;
  return "code " + std::to_string(s.code) + (msg[0] ? std::string(": ") + msg : std::string());
}

}  // namespace

extern "C" {

void* ogb_ophost_load(const char* path, char* err, int err_cap) {
  void* lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!lib) {
    set_err(err, err_cap, std::string("cannot load ") + path + ": " + dlerror());
    return nullptr;
  }
  auto negotiate = reinterpret_cast<decltype(&OgbOpNegotiate)>(dlsym(lib, "OgbOpNegotiate"));
  auto create = reinterpret_cast<decltype(&OgbOpCreateProvider)>(dlsym(lib, "OgbOpCreateProvider"));
  if (!negotiate || !create) {
    set_err(err, err_cap, std::string(path) + " does not export OgbOpNegotiate and OgbOpCreateProvider");
    dlclose(lib);
    return nullptr;
  }
  OgbOpVersion host{sizeof(OgbOpVersion), OGB_OP_ABI_MAJOR, OGB_OP_ABI_MINOR, OGB_OP_CAP_KNOWN_MASK};
  OgbOpVersion theirs{sizeof(OgbOpVersion), 0, 0, 0};
  OgbOpStatus st = negotiate(&host, &theirs);
  if (st.code != OGB_OP_OK || theirs.major != OGB_OP_ABI_MAJOR) {
    set_err(err, err_cap, "version negotiation failed: host speaks " + std::to_string(OGB_OP_ABI_MAJOR) + "." + std::to_string(OGB_OP_ABI_MINOR) +
                              ", plugin answers " + std::to_string(theirs.major) + "." + std::to_string(theirs.minor) + " (" + describe(st) + ")");
    dlclose(lib);
    return nullptr;
  }
  if (theirs.capabilities & ~OGB_OP_CAP_KNOWN_MASK) {
    char bits[32];
    std::snprintf(bits, sizeof bits, "0x%x", theirs.capabilities & ~OGB_OP_CAP_KNOWN_MASK);
    set_err(err, err_cap, std::string("the plugin needs capability bits this host does not know (") + bits + "); refusing to load it");
    dlclose(lib);
    return nullptr;
  }
  const uint32_t negotiated = std::min<uint32_t>(theirs.minor, OGB_OP_ABI_MINOR);
  OgbOpProvider filled;
  std::memset(&filled, 0, sizeof filled);
  filled.struct_size = sizeof filled;
  st = create(negotiated, &filled);
  if (st.code != OGB_OP_OK) {
    set_err(err, err_cap, "the plugin could not create a provider (" + describe(st) + ")");
    dlclose(lib);
    return nullptr;
  }
  OpPlugin* p = new (std::nothrow) OpPlugin();
  if (!p) {
    if (filled.release) filled.release(filled.self);
    dlclose(lib);
    set_err(err, err_cap, "out of memory");
    return nullptr;
  }
  std::memcpy(&p->vt, &filled, std::min<size_t>(filled.struct_size, sizeof p->vt));
  auto fail = [&](const std::string& why) -> void* {
    set_err(err, err_cap, why);
    if (p->vt.release && filled.struct_size >= sizeof(OgbOpProvider)) p->vt.release(p->vt.self);
    dlclose(lib);
    delete p;
    return nullptr;
  };
  if (filled.struct_size < sizeof(OgbOpProvider))
    return fail("the plugin's provider is " + std::to_string(filled.struct_size) + " bytes, the baseline of minor 0 is " +
                std::to_string(sizeof(OgbOpProvider)));
  if (!p->vt.kernel_count || !p->vt.kernel_desc || !p->vt.create_kernel || !p->vt.release)
    return fail("the plugin's provider lacks kernel_count, kernel_desc, create_kernel or release");
  if (p->vt.abi_minor > negotiated)
    return fail("the plugin's provider claims minor " + std::to_string(p->vt.abi_minor) + " above the negotiated " + std::to_string(negotiated));
  uint32_t n = 0;
  st = p->vt.kernel_count(p->vt.self, &n);
  if (st.code != OGB_OP_OK || n > 4096) return fail("kernel_count failed (" + describe(st) + ")");
  for (uint32_t i = 0; i < n; ++i) {
    OgbOpKernelDesc d;
    std::memset(&d, 0, sizeof d);
    d.struct_size = sizeof d;
    st = p->vt.kernel_desc(p->vt.self, i, &d);
    if (st.code != OGB_OP_OK || !d.op_type || !d.op_type[0] || !d.domain)
      return fail("kernel_desc(" + std::to_string(i) + ") failed or gave no operator name (" + describe(st) + ")");
    if (d.domain[0] == 0 && !(theirs.capabilities & OGB_OP_CAP_OVERRIDE))
      return fail(std::string("kernel '") + d.op_type + "' replaces a default-domain operator but the plugin did not ask for the override capability");
    for (const auto& seen : p->kernels)
      if (std::strcmp(seen.domain, d.domain) == 0 && std::strcmp(seen.op_type, d.op_type) == 0 && seen.since_version == d.since_version)
        return fail(std::string("the plugin lists ") + d.domain + "::" + d.op_type + " twice for the same opset");
    p->kernels.push_back(d);
  }
  p->lib = lib;
  p->capabilities = theirs.capabilities;
  return p;
}

const char* ogb_ophost_name(void* h) { return h && static_cast<OpPlugin*>(h)->vt.name ? static_cast<OpPlugin*>(h)->vt.name : ""; }
int ogb_ophost_kernel_count(void* h) { return h ? static_cast<int>(static_cast<OpPlugin*>(h)->kernels.size()) : -1; }
int ogb_ophost_capabilities(void* h) { return h ? static_cast<int>(static_cast<OpPlugin*>(h)->capabilities) : -1; }

// Writes "domain\0op_type\0" into buf; returns since_version, or -1.
int ogb_ophost_kernel_desc(void* h, int index, char* buf, int cap) {
  OpPlugin* p = static_cast<OpPlugin*>(h);
  if (!p || index < 0 || index >= static_cast<int>(p->kernels.size()) || !buf || cap < 4) return -1;
  const OgbOpKernelDesc& d = p->kernels[index];
  const size_t nd = std::strlen(d.domain), no = std::strlen(d.op_type);
  if (static_cast<int>(nd + no + 2) > cap) return -1;
  std::memcpy(buf, d.domain, nd + 1);
  std::memcpy(buf + nd + 1, d.op_type, no + 1);
  return d.since_version;
}

// `node` is an OgbOpNode prepared by the caller (attributes included, when the plugin negotiated OGB_OP_CAP_ATTRIBUTES).
void* ogb_ophost_create_kernel(void* h, int index, const OgbOpNode* node, char* err, int err_cap) {
  OpPlugin* p = static_cast<OpPlugin*>(h);
  if (!p || !node || index < 0 || index >= static_cast<int>(p->kernels.size())) {
    set_err(err, err_cap, "bad plugin handle, node or kernel index");
    return nullptr;
  }
  OgbOpNode local = *node;
  if (!(p->capabilities & OGB_OP_CAP_ATTRIBUTES)) { local.attrs = nullptr; local.num_attrs = 0; }
  OgbOpKernel filled;
  std::memset(&filled, 0, sizeof filled);
  filled.struct_size = sizeof filled;
  OgbOpStatus st = p->vt.create_kernel(p->vt.self, static_cast<uint32_t>(index), &local, &filled);
  if (st.code != OGB_OP_OK) {
    set_err(err, err_cap, describe(st));
    return nullptr;
  }
  if (filled.struct_size < sizeof(OgbOpKernel) || !filled.infer_outputs || !filled.compute || !filled.release) {
    set_err(err, err_cap, "the plugin's kernel vtable is short or lacks infer_outputs, compute or release");
    if (filled.struct_size >= sizeof(OgbOpKernel) && filled.release) filled.release(filled.self);
    return nullptr;
  }
  OpKernel* k = new (std::nothrow) OpKernel();
  if (!k) {
    filled.release(filled.self);
    set_err(err, err_cap, "out of memory");
    return nullptr;
  }
  k->owner = p;
  k->vt = filled;
  p->live_kernels += 1;
  return k;
}

// phase 0: infer_outputs (outputs' dtype / rank / dims are written), phase 1: compute.  0 on success, else an OgbOpCode.
int ogb_ophost_run(void* kh, int phase, const OgbOpTensor* inputs, int num_inputs, OgbOpTensor* outputs, int num_outputs, char* err,
                   int err_cap) {
  OpKernel* k = static_cast<OpKernel*>(kh);
  if (!k || num_inputs < 0 || num_outputs < 0 || (num_inputs && !inputs) || (num_outputs && !outputs)) return OGB_OP_INVALID_ARGUMENT;
  OgbOpStatus st = (phase == 0 ? k->vt.infer_outputs : k->vt.compute)(k->vt.self, inputs, static_cast<uint32_t>(num_inputs), outputs,
                                                                      static_cast<uint32_t>(num_outputs));
  if (st.code != OGB_OP_OK) {
    set_err(err, err_cap, describe(st));
    return static_cast<int>(st.code);
  }
  if (phase == 0) {
    for (int i = 0; i < num_outputs; ++i) {
      if (outputs[i].rank < 0 || outputs[i].rank > OGB_OP_MAX_RANK) {
        set_err(err, err_cap, "the plugin inferred output " + std::to_string(i) + " with rank " + std::to_string(outputs[i].rank));
        return OGB_OP_INTERNAL;
      }
      for (int d = 0; d < outputs[i].rank; ++d)
        if (outputs[i].dims[d] < 0) {
          set_err(err, err_cap, "the plugin inferred a negative extent for output " + std::to_string(i));
          return OGB_OP_INTERNAL;
        }
    }
  }
  return 0;
}

void ogb_ophost_release_kernel(void* kh) {
  OpKernel* k = static_cast<OpKernel*>(kh);
  if (!k) return;
  k->vt.release(k->vt.self);
  if (k->owner->live_kernels) k->owner->live_kernels -= 1;
  delete k;
}

// Refuses (returns the live count) while kernels created from the plugin are outstanding.
int ogb_ophost_unload(void* h, char* err, int err_cap) {
  OpPlugin* p = static_cast<OpPlugin*>(h);
  if (!p) return 0;
  if (p->live_kernels) {
    set_err(err, err_cap, std::to_string(p->live_kernels) + " kernel(s) of this plugin are still alive; release them first");
    return p->live_kernels;
  }
  p->vt.release(p->vt.self);
  dlclose(p->lib);
  delete p;
  return 0;
}

}  // extern "C"
