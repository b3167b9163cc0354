// NVFP4 GEMV entry point that never touches the CUDA allocator.
//
// qllm_k_nvfp4_gemv needs a caller-provided device workspace for the quantised activations.
// Some hosts cannot provide one at call time: a serving runtime that handed every byte of
// device memory to its own pool at start-up, or a thread that holds a lock under which a
// cudaMalloc/cudaFree (which synchronise the device) would stall every other stream.  For those
// callers this variant keeps the workspace in a fixed array inside the library image.
//
// * The array is shared by every call on a device: two calls that overlap in time (different
//   streams or threads) race on it.  Calls on one stream are ordered and safe.
// * Nothing in it has to start at zero: every call overwrites the part it reads.
// * The first call on a device looks the array's address up (cudaGetSymbolAddress); make that
//   first call during start-up, before any stream capture is begun on that device and before the
//   host's pool takes the rest of the device memory (the module that holds the array is loaded,
//   and the array allocated, by that first look-up).  The cached address does not survive a
//   device reset.
// * Requests that need more than kScratchBytes are rejected with QLLM_INVALID_ARGUMENT.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace qllm {

namespace {

constexpr size_t kScratchBytes = 2U << 20U;  // 2 MiB: e.g. 64 rows of 17408 columns (INT8 + block scales)
static __device__ __align__(256) uint8_t g_gemv_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_address[kMaxDevices] = {};  // several threads may make the first call

// Address of the array on the current device, looked up once per device.
int scratch_for_current_device(void** out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return check_cuda(e, "current device of the static GEMV scratch");
  if (device < 0 || device >= kMaxDevices) return fail(QLLM_INVALID_ARGUMENT, "device index beyond the static scratch table");
  void* address = g_scratch_address[device].load(std::memory_order_acquire);
  if (!address) {
    e = cudaGetSymbolAddress(&address, g_gemv_scratch);
    if (e != cudaSuccess) return check_cuda(e, "address of the static GEMV scratch");
    g_scratch_address[device].store(address, std::memory_order_release);  // every thread finds the same value
  }
  *out = address;
  return 0;
}

}  // namespace

}  // namespace qllm

using namespace qllm;

extern "C" {

size_t qllm_k_nvfp4_gemv_static_scratch_bytes(void) { return kScratchBytes; }

int qllm_k_nvfp4_gemv_static(const qllm_matrix* m, uint32_t first_row, uint32_t row_count, const float* x,
                             float* y, uint32_t batch, void* stream) {
  if (!m || !x || !y || !m->codes || !m->scales || !batch || !row_count || !m->rows || !m->cols ||
      m->cols % 16U || row_count > m->rows || first_row > m->rows - row_count || !(m->weight_scale > 0.0F) ||
      !(m->input_scale > 0.0F))
    return fail(QLLM_INVALID_ARGUMENT, "invalid native NVFP4 GEMV");
  // the kernels read x as float4, the codes as uint2 and the scales of a row as whole words
  if ((reinterpret_cast<uintptr_t>(x) & 15U) || (reinterpret_cast<uintptr_t>(m->codes) & 7U))
    return fail(QLLM_INVALID_ARGUMENT, "native NVFP4 GEMV needs x on a 16-byte and the codes on an 8-byte boundary");
  const size_t need = act_quant_bytes(batch, m->cols);
  if (need > kScratchBytes)
    return fail(QLLM_INVALID_ARGUMENT,
                "batch x columns needs " + std::to_string(need) + " bytes of scratch; the static array holds " +
                    std::to_string(kScratchBytes) + " (use qllm_k_nvfp4_gemv with a workspace)");
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  auto s = static_cast<cudaStream_t>(stream);
  rc = launch_act_quant_i8(x, scratch, batch, m->cols, m->input_scale, s);
  if (rc) return rc;
  return launch_gemv_simt(*m, first_row, row_count, scratch, batch, y, batch, s);
}

}  // extern "C"
