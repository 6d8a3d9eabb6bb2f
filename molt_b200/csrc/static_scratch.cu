// molt_nf4_lora_fwd_static: the NF4-LoRA forward for callers that are not able to hand over scratch memory.
//
// Who needs this: a host that drives the library from a context in which it cannot call cudaMalloc (or any
// allocating routine, a framework's caching allocator included) -- for example an inference server that pins its
// whole device budget at start-up and forbids later allocations, a plugin loaded into a process whose allocator it
// does not own, or code running between the capture-safe parts of somebody else's step.  The regular entry point
// molt_nf4_lora_fwd asks the caller for a workspace; this one brings its own, a fixed array that is part of the
// library's device image.
//
// Cost and limits: every GPU that loads the library holds kStaticScratchBytes (16 MiB) until the process exits.
// Problem sizes whose forward scratch exceeds that are refused with MOLT_E_VALUE.  All calls on one device share
// the array, and it keeps whatever the previous call left in it.  Nothing in the forward relies on zeroed scratch
// (every buffer carved from it is fully written before it is read), so no clearing is needed between calls -- but
// two calls whose kernels can overlap on the GPU (different streams without an ordering between them) race on
// it.  Serialise such calls.
//
// Set-up: the first call on a device asks the runtime for the array's device address (cudaGetSymbolAddress, with
// that device current) and remembers it.  Make that first call outside of any stream capture.
#include <mutex>

#include "internal.h"

namespace molt {
namespace {

constexpr size_t kStaticScratchBytes = MOLT_STATIC_SCRATCH_BYTES;

// The scratch itself.  In host code this name is only a handle for the runtime, not a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_address[64] = {nullptr};

// Device address of the array on the calling thread's current device, looked up once per device.
int scratch_address(void** out) {
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MOLT_E_CAPABILITY, "molt_nf4_lora_fwd_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr)
      return fail(MOLT_E_RUNTIME, "molt_nf4_lora_fwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
    g_scratch_address[dev] = ptr;
  }
  *out = g_scratch_address[dev];
  return MOLT_OK;
}

}  // namespace
}  // namespace molt

using namespace molt;

extern "C" int molt_nf4_lora_fwd_static(const molt_nf4_desc* w, const void* x, const float* lora_a,
                                        const float* lora_b, float scaling, int rank, void* y, int64_t m, int path,
                                        uintptr_t stream) {
  MOLT_REQUIRE(w != nullptr, MOLT_E_VALUE, "molt_nf4_lora_fwd_static: weight descriptor is NULL");
  MOLT_REQUIRE(rank <= 64, MOLT_E_CAPABILITY, "molt_nf4_lora_fwd_static: LoRA rank %d exceeds the supported maximum of 64",
               rank);
  // the smallest workspace the forward accepts (without the optional scratch of the tensor-core kernel's split schedule)
  const size_t need = workspace_bytes(MOLT_OP_LORA_FWD, m, w->n, w->k, rank, false);
  MOLT_REQUIRE(need != 0, MOLT_E_VALUE, "molt_nf4_lora_fwd_static: invalid sizes (m=%lld n=%lld k=%lld rank=%d)",
               (long long)m, (long long)w->n, (long long)w->k, rank);
  MOLT_REQUIRE(need <= kStaticScratchBytes, MOLT_E_VALUE,
               "molt_nf4_lora_fwd_static: this problem needs %zu bytes of scratch but the built-in scratch holds %zu; "
               "use molt_nf4_lora_fwd with a caller-provided workspace",
               need, kStaticScratchBytes);
  void* scratch = nullptr;
  if (int rc = scratch_address(&scratch)) return rc;
  return molt_nf4_lora_fwd(w, x, lora_a, lora_b, scaling, rank, y, m, nullptr, scratch, kStaticScratchBytes, path,
                           stream);
}
