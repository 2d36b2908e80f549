/*
 * Operator plugin ABI: a shared library that brings kernels for ONNX operators -- new ones in its own domain, or
 * replacements for built-in ones -- to the graph executor without linking against it.  This header is the whole
 * contract; a plugin may be written in C.  Role of the reference's native execution-provider plugin ABI
 * (crates/onnx-runtime-ep-nxrt-abi/src/lib.rs:1-60, vtable.rs): two exported symbols, a version handshake that fails
 * closed (wrong major or an unknown capability bit is a refusal, never a guess), every struct starts with its own size
 * so that fields can be appended, explicit ownership (borrowed pointers live for the call, owned objects have a
 * release slot in their vtable), and status codes instead of exceptions.
 *
 * Exported by a plugin:
 *   OgbOpNegotiate        agree on a version and on capability bits
 *   OgbOpCreateProvider   fill a provider vtable (kernel registry + kernel factory)
 *
 * Flow on the host: negotiate -> create provider -> enumerate kernel descriptions -> for a node of the graph that
 * matches a description: create_kernel (the plugin sees the node's attributes once) -> per call: infer_outputs (shapes
 * and element types from the input descriptions), the host allocates the outputs, compute -> release the kernel ->
 * release the provider.  Tensors are dense, row-major, in host memory.
 *
 * Reading rule for both sides: read struct_size first; copy min(struct_size, sizeof(local)) bytes into a zeroed local;
 * reject a struct smaller than the baseline of the minor version it claims; never call a slot beyond the copied prefix.
 */
#ifndef OGB_KERNEL_ABI_H
#define OGB_KERNEL_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OGB_OP_ABI_MAJOR 1u
#define OGB_OP_ABI_MINOR 0u
#define OGB_OP_MAX_RANK 8

/* capability bits a plugin may ask the host for; the host refuses bits it does not know */
#define OGB_OP_CAP_ATTRIBUTES 0x1u   /* the plugin reads node attributes */
#define OGB_OP_CAP_OVERRIDE 0x2u     /* the plugin replaces built-in operators of the default domain */
#define OGB_OP_CAP_KNOWN_MASK 0x3u

typedef enum OgbOpCode {
  OGB_OP_OK = 0,
  OGB_OP_INVALID_ARGUMENT = 1,
  OGB_OP_UNSUPPORTED = 2,
  OGB_OP_VERSION_MISMATCH = 3,
  OGB_OP_INTERNAL = 4
} OgbOpCode;

typedef struct OgbOpStatus {
  uint32_t struct_size;
  uint32_t code;     /* OgbOpCode */
  char message[120]; /* NUL-terminated, may be empty */
} OgbOpStatus;

typedef struct OgbOpVersion {
  uint32_t struct_size;
  uint32_t major;
  uint32_t minor;
  uint32_t capabilities; /* host -> plugin: bits the host knows; plugin -> host: bits the plugin needs */
} OgbOpVersion;

/* element types: the values of onnx.TensorProto.DataType (1 float32, 7 int64, 9 bool, 10 float16, 11 float64, ...) */
typedef struct OgbOpTensor {
  uint32_t struct_size;
  int32_t dtype;
  int32_t rank;
  int32_t reserved;
  int64_t dims[OGB_OP_MAX_RANK];
  void* data;         /* NULL in descriptions passed to infer_outputs; borrowed for the call in compute */
  uint64_t byte_size;
} OgbOpTensor;

typedef enum OgbOpAttrKind { OGB_OP_ATTR_INT = 1, OGB_OP_ATTR_FLOAT = 2, OGB_OP_ATTR_STRING = 3, OGB_OP_ATTR_INTS = 4, OGB_OP_ATTR_FLOATS = 5 } OgbOpAttrKind;

typedef struct OgbOpAttr {
  uint32_t struct_size;
  uint32_t kind;       /* OgbOpAttrKind */
  const char* name;    /* borrowed for the call */
  uint64_t count;      /* elements of ints / floats, bytes of string, 1 otherwise */
  const int64_t* ints; /* INT, INTS */
  const double* floats;/* FLOAT, FLOATS */
  const char* string;  /* STRING (not necessarily NUL-terminated: use count) */
} OgbOpAttr;

typedef struct OgbOpNode {
  uint32_t struct_size;
  uint32_t num_attrs;
  const char* domain;  /* "" for the default domain */
  const char* op_type;
  const char* name;    /* may be empty */
  const OgbOpAttr* attrs;
  uint32_t num_inputs, num_outputs;
} OgbOpNode;

typedef struct OgbOpKernelDesc {
  uint32_t struct_size;
  int32_t since_version; /* lowest opset of the domain this kernel serves */
  const char* domain;    /* static strings owned by the plugin */
  const char* op_type;
} OgbOpKernelDesc;

typedef struct OgbOpKernel {
  uint32_t struct_size;
  uint32_t reserved;
  void* self;
  /* outputs[i].dtype / rank / dims are written by the plugin; data stays NULL */
  OgbOpStatus (*infer_outputs)(void* self, const OgbOpTensor* inputs, uint32_t num_inputs, OgbOpTensor* outputs, uint32_t num_outputs);
  OgbOpStatus (*compute)(void* self, const OgbOpTensor* inputs, uint32_t num_inputs, OgbOpTensor* outputs, uint32_t num_outputs);
  void (*release)(void* self);
} OgbOpKernel;

typedef struct OgbOpProvider {
  uint32_t struct_size;
  uint32_t abi_minor;
  void* self;
  const char* name;     /* static string owned by the plugin */
  OgbOpStatus (*kernel_count)(void* self, uint32_t* out_count);
  OgbOpStatus (*kernel_desc)(void* self, uint32_t index, OgbOpKernelDesc* out);
  OgbOpStatus (*create_kernel)(void* self, uint32_t index, const OgbOpNode* node, OgbOpKernel* out);
  void (*release)(void* self);
} OgbOpProvider;

#if defined(_WIN32)
#define OGB_OP_EXPORT __declspec(dllexport)
#else
#define OGB_OP_EXPORT __attribute__((visibility("default")))
#endif

OGB_OP_EXPORT OgbOpStatus OgbOpNegotiate(const OgbOpVersion* host, OgbOpVersion* plugin);
OGB_OP_EXPORT OgbOpStatus OgbOpCreateProvider(uint32_t negotiated_minor, OgbOpProvider* out);

#ifdef __cplusplus
}
#endif
#endif
