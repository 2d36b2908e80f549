// Growable host buffers: reserve an address range once, commit pages behind its front as it grows, give pages back as
// it shrinks, never move the base.  Host-side counterpart of the device VMM pool (csrc/kernels/vmm_pool.cu) and of the
// reference's reserve-and-map host buffers (crates/onnx-runtime-virtual-memory/src/buffer.rs, sys.rs).  POSIX: the range
// is an anonymous PROT_NONE mapping; commit = mprotect(READ|WRITE); decommit = madvise(DONTNEED) + PROT_NONE, which
// returns the physical pages and makes a stale access fault at once instead of reading zeros.
#include <sys/mman.h>
#include <unistd.h>

#include <cerrno>
#include <cstdint>
#include <cstring>

namespace {
struct HostRange {
  uint8_t* base;
  uint64_t reserved, committed, page;
};
uint64_t round_up(uint64_t v, uint64_t g) { return (v + g - 1) / g * g; }
}  // namespace

extern "C" {

void* ogb_hostvmm_reserve(uint64_t bytes) {
  const uint64_t page = static_cast<uint64_t>(sysconf(_SC_PAGESIZE));
  const uint64_t size = round_up(bytes ? bytes : 1, page);
  void* p = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (p == MAP_FAILED) return nullptr;
  return new HostRange{static_cast<uint8_t*>(p), size, 0, page};
}

// Make at least `bytes` from the start usable (page-rounded).  Returns 0, or errno; -1 when beyond the reservation.
int ogb_hostvmm_commit(void* h, uint64_t bytes) {
  HostRange* r = static_cast<HostRange*>(h);
  if (!r) return EINVAL;
  const uint64_t want = round_up(bytes, r->page);
  if (want > r->reserved) return -1;
  if (want <= r->committed) return 0;
  if (mprotect(r->base + r->committed, want - r->committed, PROT_READ | PROT_WRITE) != 0) return errno;
  r->committed = want;
  return 0;
}

// Keep the first `bytes` (page-rounded up); return the rest to the system.
int ogb_hostvmm_decommit(void* h, uint64_t bytes) {
  HostRange* r = static_cast<HostRange*>(h);
  if (!r) return EINVAL;
  const uint64_t keep = round_up(bytes, r->page);
  if (keep >= r->committed) return 0;
  if (madvise(r->base + keep, r->committed - keep, MADV_DONTNEED) != 0) return errno;
  if (mprotect(r->base + keep, r->committed - keep, PROT_NONE) != 0) return errno;
  r->committed = keep;
  return 0;
}

uint64_t ogb_hostvmm_base(void* h) { return h ? reinterpret_cast<uint64_t>(static_cast<HostRange*>(h)->base) : 0; }
uint64_t ogb_hostvmm_committed(void* h) { return h ? static_cast<HostRange*>(h)->committed : 0; }
uint64_t ogb_hostvmm_reserved(void* h) { return h ? static_cast<HostRange*>(h)->reserved : 0; }
uint64_t ogb_hostvmm_page(void* h) { return h ? static_cast<HostRange*>(h)->page : 0; }

void ogb_hostvmm_release(void* h) {
  HostRange* r = static_cast<HostRange*>(h);
  if (!r) return;
  munmap(r->base, r->reserved);
  delete r;
}

}  // extern "C"
