/*
 * Example operator plugin (csrc/abi/ogb_kernel_abi.h).  Two kernels:
 *   example.ops::ScaledClip   y = clip(alpha * x, lo, hi) for float32 tensors; attributes alpha (float), lo, hi (float)
 *   ::Relu                    a replacement for the built-in Relu that counts its calls (needs the override capability)
 *
 * Build:  cc -shared -fPIC -I csrc examples/plugins/example_ops.c -o libexample_ops.so
 * Compile-time switches produce the misbehaving variants the tests load:
 *   -DOGB_OP_WRONG_MAJOR      answers the handshake with major 2
 *   -DOGB_OP_UNKNOWN_CAP      asks for a capability bit no host knows
 *   -DOGB_OP_SHORT_VTABLE     fills a provider smaller than the baseline
 *   -DOGB_OP_NO_OVERRIDE_CAP  lists ::Relu without asking for the override capability
 *   -DOGB_OP_FAILING_KERNEL   ScaledClip's compute reports an error
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "abi/ogb_kernel_abi.h"

static OgbOpStatus status(uint32_t code, const char* msg) {
  OgbOpStatus s;
  memset(&s, 0, sizeof s);
  s.struct_size = sizeof s;
  s.code = code;
  if (msg) snprintf(s.message, sizeof s.message, "%s", msg);
  return s;
}

typedef struct Clip { float alpha, lo, hi; } Clip;
static long g_relu_calls = 0;
OGB_OP_EXPORT long example_ops_relu_calls(void) { return g_relu_calls; }

static OgbOpStatus same_as_input(void* self, const OgbOpTensor* in, uint32_t n_in, OgbOpTensor* out, uint32_t n_out) {
  (void)self;
  if (n_in != 1 || n_out != 1) return status(OGB_OP_INVALID_ARGUMENT, "one input and one output expected");
  if (in[0].dtype != 1) return status(OGB_OP_UNSUPPORTED, "float32 only");
  out[0].dtype = in[0].dtype;
  out[0].rank = in[0].rank;
  memcpy(out[0].dims, in[0].dims, sizeof in[0].dims);
  return status(OGB_OP_OK, NULL);
}

static OgbOpStatus clip_compute(void* self, const OgbOpTensor* in, uint32_t n_in, OgbOpTensor* out, uint32_t n_out) {
  const Clip* c = (const Clip*)self;
  (void)n_in; (void)n_out;
#ifdef OGB_OP_FAILING_KERNEL
  (void)c; (void)in; (void)out;
  return status(OGB_OP_INTERNAL, "ScaledClip: device lost (injected)");
#else
  const float* x = (const float*)in[0].data;
  float* y = (float*)out[0].data;
  const uint64_t n = in[0].byte_size / sizeof(float);
  if (out[0].byte_size != in[0].byte_size) return status(OGB_OP_INVALID_ARGUMENT, "output buffer has the wrong size");
  for (uint64_t i = 0; i < n; ++i) {
    float v = c->alpha * x[i];
    y[i] = v < c->lo ? c->lo : (v > c->hi ? c->hi : v);
  }
  return status(OGB_OP_OK, NULL);
#endif
}

static OgbOpStatus relu_compute(void* self, const OgbOpTensor* in, uint32_t n_in, OgbOpTensor* out, uint32_t n_out) {
  (void)self; (void)n_in; (void)n_out;
  const float* x = (const float*)in[0].data;
  float* y = (float*)out[0].data;
  const uint64_t n = in[0].byte_size / sizeof(float);
  for (uint64_t i = 0; i < n; ++i) y[i] = x[i] > 0.f ? x[i] : 0.f;
  ++g_relu_calls;
  return status(OGB_OP_OK, NULL);
}

static void free_self(void* self) { free(self); }
static void no_release(void* self) { (void)self; }

static OgbOpStatus kernel_count(void* self, uint32_t* out) { (void)self; *out = 2; return status(OGB_OP_OK, NULL); }

static OgbOpStatus kernel_desc(void* self, uint32_t i, OgbOpKernelDesc* out) {
  (void)self;
  if (i > 1) return status(OGB_OP_INVALID_ARGUMENT, "no such kernel");
  out->since_version = i == 0 ? 1 : 6;
  out->domain = i == 0 ? "example.ops" : "";
  out->op_type = i == 0 ? "ScaledClip" : "Relu";
  return status(OGB_OP_OK, NULL);
}

static OgbOpStatus create_kernel(void* self, uint32_t i, const OgbOpNode* node, OgbOpKernel* out) {
  (void)self;
  if (out->struct_size < sizeof(OgbOpKernel)) return status(OGB_OP_INVALID_ARGUMENT, "kernel struct too small");
  out->struct_size = sizeof(OgbOpKernel);
  out->infer_outputs = same_as_input;
  if (i == 1) {
    out->self = NULL;
    out->compute = relu_compute;
    out->release = no_release;
    return status(OGB_OP_OK, NULL);
  }
  Clip* c = (Clip*)malloc(sizeof(Clip));
  if (!c) return status(OGB_OP_INTERNAL, "out of memory");
  c->alpha = 1.f; c->lo = -1.f; c->hi = 1.f;
  for (uint32_t a = 0; a < node->num_attrs; ++a) {
    const OgbOpAttr* at = &node->attrs[a];
    if (at->kind != OGB_OP_ATTR_FLOAT || !at->floats) continue;
    if (strcmp(at->name, "alpha") == 0) c->alpha = (float)at->floats[0];
    if (strcmp(at->name, "lo") == 0) c->lo = (float)at->floats[0];
    if (strcmp(at->name, "hi") == 0) c->hi = (float)at->floats[0];
  }
  if (c->lo > c->hi) { free(c); return status(OGB_OP_INVALID_ARGUMENT, "ScaledClip: lo exceeds hi"); }
  out->self = c;
  out->compute = clip_compute;
  out->release = free_self;
  return status(OGB_OP_OK, NULL);
}

OGB_OP_EXPORT OgbOpStatus OgbOpNegotiate(const OgbOpVersion* host, OgbOpVersion* plugin) {
  plugin->struct_size = sizeof *plugin;
#ifdef OGB_OP_WRONG_MAJOR
  plugin->major = 2;
#else
  plugin->major = OGB_OP_ABI_MAJOR;
#endif
  plugin->minor = 0;
  plugin->capabilities = OGB_OP_CAP_ATTRIBUTES;
#ifndef OGB_OP_NO_OVERRIDE_CAP
  plugin->capabilities |= OGB_OP_CAP_OVERRIDE;
#endif
#ifdef OGB_OP_UNKNOWN_CAP
  plugin->capabilities |= 0x100u;
#endif
  if (host->major != plugin->major) return status(OGB_OP_VERSION_MISMATCH, "this plugin speaks another major version");
  return status(OGB_OP_OK, NULL);
}

OGB_OP_EXPORT OgbOpStatus OgbOpCreateProvider(uint32_t negotiated_minor, OgbOpProvider* out) {
  (void)negotiated_minor;
#ifdef OGB_OP_SHORT_VTABLE
  out->struct_size = 24;
  return status(OGB_OP_OK, NULL);
#else
  if (out->struct_size < sizeof(OgbOpProvider)) return status(OGB_OP_INVALID_ARGUMENT, "provider struct too small");
  out->struct_size = sizeof(OgbOpProvider);
  out->abi_minor = 0;
  out->self = NULL;
  out->name = "example-ops";
  out->kernel_count = kernel_count;
  out->kernel_desc = kernel_desc;
  out->create_kernel = create_kernel;
  out->release = no_release;
  return status(OGB_OP_OK, NULL);
#endif
}
