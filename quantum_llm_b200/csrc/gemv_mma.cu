// NVFP4 x NVFP4 skinny GEMM on the 5th-generation tensor cores (sm_100a).
//
// The reference's W4A4 GEMV fake-quantises the activations to E2M1 with one E4M3 scale
// per 16 values, i.e. both operands are NVFP4, which is exactly what
// tcgen05.mma.kind::mxf4nvf4.block_scale computes.  The weights are the M operand
// (128 weight rows per CTA), the activation rows are the N operand (padded to 16..128),
// so the weight stream goes HBM -> TMA -> shared memory -> tensor core without passing
// through registers; the kernel is judged by the HBM bandwidth it sustains.
//
//   D[row, j] = sum_blocks (sum_i cw_i * cx_i) * sw * sx      (FP32 in tensor memory)
//   y[j, row] = bf16(D * weight_scale / input_scale)
//
// Layouts: codes stay as the checkpoint has them ([rows, K/2], low nibble = even k) and
// are fetched by a 128B-swizzled 2D TMA box of 128 rows x 256 k.  The E4M3 block scales
// are re-tiled once at load time into 512-byte atoms (128 rows x 4 blocks:
// offset = (row%32)*16 + (row/32)*4 + block%4), the form tcgen05.cp.32x128b.warpx4
// moves into tensor memory.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "fused.h"
#include "gemv_mma.h"
#include "launch.cuh"
#include "rope_tail.cuh"

namespace qllm {

namespace {

constexpr uint32_t kTileRows = 128;    // weight rows per CTA (UMMA M)
constexpr uint32_t kTileK = 256;       // k values per pipeline stage (128 bytes of codes per row)
constexpr uint32_t kAtomBytes = 512;   // scale atom: 128 rows x 4 blocks
constexpr uint32_t kABytes = kTileRows * kTileK / 2;   // 16 KB
constexpr uint32_t kSfBytes = (kTileK / 64) * kAtomBytes;  // 2 KB per operand per stage
constexpr uint32_t kSpinLimit = 1U << 20;

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);

// scale atoms (64 k values each) of a row tile, padded to whole 256-wide pipeline stages
__host__ __device__ inline uint32_t padded_atoms(uint32_t cols) { return (cols + kTileK - 1U) / kTileK * (kTileK / 64U); }
inline uint32_t k_chunks_of(uint32_t cols) { return (cols + kTileK - 1U) / kTileK; }

EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  });
  return fn;
}

// 2D map over packed codes: [rows, k_bytes] bytes, box = [box_rows, 128 bytes], 128B swizzle.
int make_codes_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k_bytes, uint32_t box_rows) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return fail(QLLM_INTERNAL, "cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[2] = {k_bytes, rows};
  const cuuint64_t strides[1] = {k_bytes};
  const cuuint32_t box[2] = {128U, box_rows};
  const cuuint32_t elem[2] = {1U, 1U};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QLLM_INTERNAL, "cuTensorMapEncodeTiled failed (" + std::to_string(r) + ")");
  return 0;
}

// [rows, K/16] row-major scale bytes -> [row_tile][k_atom][512] atoms.
__global__ void retile_scales_kernel(const uint8_t* __restrict__ scales, uint8_t* __restrict__ tiled,
                                     uint32_t rows, uint32_t blocks, uint32_t k_atoms) {
  const uint64_t item = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const uint32_t row_tiles = (rows + kTileRows - 1U) / kTileRows;
  const uint64_t total = static_cast<uint64_t>(row_tiles) * k_atoms * (kAtomBytes / 4U);
  if (item >= total) return;
  // one thread per 4 scale bytes (the 4 blocks of one row in one atom)
  const uint32_t within = static_cast<uint32_t>(item % (kAtomBytes / 4U));
  const uint64_t atom = item / (kAtomBytes / 4U);
  const uint32_t k_atom = static_cast<uint32_t>(atom % k_atoms);
  const uint32_t tile = static_cast<uint32_t>(atom / k_atoms);
  const uint32_t r0 = within / 4U, r1 = within % 4U;  // byte offset r0*16 + r1*4
  const uint32_t row = tile * kTileRows + r1 * 32U + r0;
  uint32_t word = 0U;
  if (row < rows) {
#pragma unroll
    for (uint32_t b = 0; b < 4U; ++b) {
      const uint32_t block = k_atom * 4U + b;
      if (block < blocks)
        word |= static_cast<uint32_t>(scales[static_cast<size_t>(row) * blocks + block] & 0x7fU) << (8U * b);
    }
  }
  reinterpret_cast<uint32_t*>(tiled)[item] = word;
}

}  // namespace

int MmaWeights::prepare(const qllm_matrix& m, cudaStream_t stream) {
  release();
  rows = m.rows;
  cols = m.cols;
  if (m.cols % 64U) return 0;  // shape outside the tensor-core path; the CUDA-core kernel serves it
  // K need not be a multiple of the 256-wide pipeline stage (a tensor-parallel K slice): the
  // re-tiled scales are padded with zeros to whole stages, the codes' last box is filled with
  // zeros by the TMA unit, and the kernel issues only the 64-wide MMAs that lie inside K
  const uint32_t blocks = m.cols / 16U, k_atoms = padded_atoms(m.cols);
  const uint32_t row_tiles = (m.rows + kTileRows - 1U) / kTileRows;
  const size_t bytes = static_cast<size_t>(row_tiles) * k_atoms * kAtomBytes;
  int rc = check_cuda(cudaMalloc(&tiled_scales, bytes), "re-tiled scale allocation");
  if (rc) return rc;
  const uint64_t items = bytes / 4U;
  retile_scales_kernel<<<static_cast<unsigned>((items + 255U) / 256U), 256, 0, stream>>>(
      m.scales, tiled_scales, m.rows, blocks, k_atoms);
  count_launch();
  rc = check_launch("retile_scales");
  if (rc) return rc;
  rc = make_codes_map(&codes_map, m.codes, m.rows, m.cols / 2U, kTileRows);
  if (rc) return rc;
  ready = true;
  return 0;
}

void MmaWeights::release() {
  if (tiled_scales) cudaFree(tiled_scales);
  tiled_scales = nullptr;
  ready = false;
}

MmaWeights& MmaWeights::operator=(MmaWeights&& o) noexcept {
  if (this != &o) {
    release();
    codes_map = o.codes_map;
    tiled_scales = o.tiled_scales;
    rows = o.rows;
    cols = o.cols;
    ready = o.ready;
    o.tiled_scales = nullptr;
    o.ready = false;
  }
  return *this;
}

// ---------------------------------------------------------------- activations
// Workspace layout (all 1024-byte aligned):
//   [error word | pad] [codes: n_pad x K/2] [scale atoms: n_tiles x k_atoms x 512] [partials]
struct MmaWorkspace {
  uint32_t* error;
  uint8_t* codes;
  uint8_t* atoms;
  float* partials;
  uint32_t n_pad, n_tiles;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1U) / a * a; }

static uint32_t pick_split(uint32_t row_tiles, uint32_t n_tiles, uint32_t k_chunks) {
  // one wave of at most two CTAs per SM (a second, partial wave costs a whole CTA's time),
  // with at least 3 k-chunks of work per CTA
  const uint32_t want = (2U * 148U) / (row_tiles * n_tiles);
  const uint32_t cap = std::max(1U, k_chunks / 3U);
  return std::max(1U, std::min(want, cap));
}

static MmaWorkspace carve(void* workspace, uint32_t batch, uint32_t rows, uint32_t cols, uint32_t split,
                          size_t* total) {
  MmaWorkspace w{};
  w.n_pad = (batch + 15U) / 16U * 16U;
  w.n_tiles = (w.n_pad + 127U) / 128U;
  uint8_t* base = static_cast<uint8_t*>(workspace);
  size_t off = 1024;
  w.error = reinterpret_cast<uint32_t*>(base);
  w.codes = base + off;
  off += align_up(static_cast<size_t>(w.n_tiles) * 128U * (cols / 2U), 1024);
  w.atoms = base + off;
  off += align_up(static_cast<size_t>(w.n_tiles) * padded_atoms(cols) * kAtomBytes, 1024);
  w.partials = reinterpret_cast<float*>(base + off);
  off += align_up(static_cast<size_t>(split) * batch * rows * sizeof(float), 1024);
  if (total) *total = off;
  return w;
}

size_t gemv_mma_workspace_bytes(uint32_t batch, uint32_t rows, uint32_t cols) {
  if (cols % 64U) return 0;
  size_t total = 0;
  const uint32_t row_tiles = (rows + kTileRows - 1U) / kTileRows;
  // the split depends on n_tiles only through its product with row_tiles; size for the worst case
  const uint32_t split = pick_split(row_tiles, 1U, k_chunks_of(cols));
  carve(nullptr, batch, rows, cols, split, &total);
  return total;
}

// One thread per (padded row, 16-value block): packed E2M1 codes (8 bytes) into the row-major
// code matrix, the E4M3 scale into its atom.  Rows past `batch` are written as zeros.
__global__ void act_quant_mma_kernel(const float* __restrict__ x, uint8_t* __restrict__ codes,
                                     uint8_t* __restrict__ atoms, uint32_t batch, uint32_t rows_total,
                                     uint32_t cols, float g) {
  const uint32_t blocks = cols / 16U;
  const uint64_t item = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= static_cast<uint64_t>(rows_total) * blocks) return;
  const uint32_t m = static_cast<uint32_t>(item / blocks), b = static_cast<uint32_t>(item % blocks);
  uint32_t packed[2] = {0U, 0U};
  unsigned sc = 0U;
  if (m < batch) {
    const float4* in4 = reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * cols + b * 16U);
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 t = in4[i];
      v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    float amax = 0.0F;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    sc = e4m3_code(fminf(448.0F, g * amax / 6.0F));
    const float local = e4m3_value(sc);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      unsigned code = 0U;
      if (local != 0.0F) code = e2m1_code(fminf(6.0F, fmaxf(-6.0F, v[i] * g / local)));
      packed[i / 8] |= code << (4 * (i % 8));
    }
  }
  reinterpret_cast<uint2*>(codes + static_cast<size_t>(m) * (cols / 2U))[b] = make_uint2(packed[0], packed[1]);
  const uint32_t tile = m / 128U, r = m % 128U;
  atoms[(static_cast<size_t>(tile) * padded_atoms(cols) + b / 4U) * kAtomBytes + (r % 32U) * 16U + (r / 32U) * 4U +
        b % 4U] = static_cast<uint8_t>(sc);
}

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait: false when the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 255U) == 255U && *abort_flag) return false;
  }
  *abort_flag = 1U;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, uint32_t x,
                                            uint32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// K-major operand tile in 128B-swizzled shared memory: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffU) >> 4U);       // start address
  d |= static_cast<uint64_t>(1U) << 16U;                       // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024U >> 4U) << 32U;              // stride byte offset
  d |= static_cast<uint64_t>(1U) << 46U;                       // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2U) << 61U;                       // SWIZZLE_128B
  return d;
}
// 32 rows x 16 bytes, unswizzled (source of tcgen05.cp.32x128b): 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sf(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffU) >> 4U);
  d |= static_cast<uint64_t>(1U) << 16U;
  d |= static_cast<uint64_t>(128U >> 4U) << 32U;
  d |= static_cast<uint64_t>(1U) << 46U;
  return d;
}

struct GemvMmaParams {
  const uint8_t* tiled_scales;  // weights: [row_tile][k_atom][512]
  const uint8_t* act_atoms;     // activations: [n_tile][k_atom][512]
  float* partials;              // [split][batch][row_count] when split > 1
  float* y;                     // [batch][row_count]
  uint32_t* error;
  uint32_t first_tile, row_count, batch, n_pad;
  uint32_t k_chunks, k_atoms, split, stages;  // k_atoms: atoms per row tile in memory (whole stages)
  uint32_t raw;                 // bit 0: always write raw partials (the consumer applies the scale);
                                // bits 1..: 64-wide k groups that lie inside K (the last stage may be partial)
  float weight_scale, input_scale;
};

// grid (row tiles, split, n tiles); 128 threads: thread 0 drives TMA, thread 32 drives the tensor
// core, all four warps run the epilogue (one tensor-memory lane = one weight row per thread).
// kExchange: the tensor-parallel form, kept out of the single-GPU instantiation together with
// its launch parameters.
template <bool kExchange> struct ExchangeParam {};
template <> struct ExchangeParam<true> { GemvExchange x; };
// kRopeTail: the fused q/k/v projection of a decode step finishes every head itself -- the CTA
// that takes the last ticket of a 128-row tile (= one head of head_dim 128) adds up the tile's
// split-K partial sums, rotates the head and stores the INT8 query or the K/V record
// (rope_tail.cuh), so no separate RoPE / KV-store kernel follows the GEMV.
template <bool kRopeTail> struct TailParam {};
template <> struct TailParam<true> { RopeTail t; };

// kPartialK: K is not a whole number of 256-wide stages (the last stage issues fewer MMAs); its own
// instantiation so that the common form carries no extra state.
template <bool kExchange, bool kPartialK, bool kRopeTail>
__global__ void __launch_bounds__(128)
nvfp4_gemv_mma_kernel(const __grid_constant__ CUtensorMap weight_map,
                      const __grid_constant__ CUtensorMap act_map, GemvMmaParams p,
                      const __grid_constant__ ExchangeParam<kExchange> e,
                      const __grid_constant__ TailParam<kRopeTail> tail) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  pdl_trigger();  // the consumer kernel may be scheduled; it waits for this grid to finish
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], done_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_word;
  __shared__ uint2* exchange_inbox[8];  // tensor parallel: this exchange's slot in every rank's inbox
  if constexpr (kExchange) {
#pragma unroll
    for (uint32_t r = 0; r < 8U; ++r)  // constant indices: the parameter struct stays in the parameter space
      if (threadIdx.x == r) exchange_inbox[r] = e.x.inbox[r];
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023U) & ~uintptr_t(1023));
  const uint32_t tid = threadIdx.x, warp = tid >> 5U;
  const uint32_t n_tile = blockIdx.z;
  const uint32_t n_rows = min(128U, p.n_pad - n_tile * 128U);  // UMMA N of this CTA (multiple of 16)
  const uint32_t b_bytes = min(p.n_pad, 128U) * 128U;          // TMA box of the activation codes
  const uint32_t stage_bytes = kABytes + kSfBytes + ((b_bytes + 1023U) & ~1023U) + kSfBytes;
  const uint32_t tile = p.first_tile + blockIdx.x;
  // k range of this split
  const uint32_t per = p.k_chunks / p.split, extra = p.k_chunks % p.split;
  const uint32_t kc0 = blockIdx.y * per + min(blockIdx.y, extra);
  const uint32_t kcn = per + (blockIdx.y < extra ? 1U : 0U);
  // tensor memory: accumulator [128 lanes x n_rows] then 16 columns of scales per operand
  const uint32_t acc_cols = n_rows < 32U ? 32U : n_rows;
  uint32_t tmem_cols = 32U;
  while (tmem_cols < acc_cols + 32U) tmem_cols <<= 1U;

  if (tid == 0U) {
    for (uint32_t s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1U); mbar_init(&empty_bar[s], 1U); }
    mbar_init(&done_bar, 1U);
    abort_word = 0U;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0U) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_base_slot;
  const uint32_t tmem_sfa = tmem_acc + acc_cols;
  const uint32_t tmem_sfb = tmem_sfa + 16U;
  volatile uint32_t* abort_flag = &abort_word;

  if (tid == 0U) {
    // ---- producer: TMA loads of weight codes, weight scales, activation codes, activation scales
    auto load_weights = [&](uint32_t i) {
      const uint32_t s = i % p.stages, kc = kc0 + i;
      uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
      mbar_expect_tx(&full_bar[s], kABytes + 2U * kSfBytes + b_bytes);
      tma_load_2d(st, &weight_map, &full_bar[s], kc * 128U, tile * kTileRows);
      bulk_load(st + kABytes, p.tiled_scales + (static_cast<size_t>(tile) * p.k_atoms + kc * 4U) * kAtomBytes,
                kSfBytes, &full_bar[s]);
    };
    auto load_activations = [&](uint32_t i) {
      const uint32_t s = i % p.stages, kc = kc0 + i;
      uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
      tma_load_2d(st + kABytes + kSfBytes, &act_map, &full_bar[s], kc * 128U, n_tile * 128U);
      bulk_load(st + stage_bytes - kSfBytes,
                p.act_atoms + (static_cast<size_t>(n_tile) * p.k_atoms + kc * 4U) * kAtomBytes, kSfBytes,
                &full_bar[s]);
    };
    // the weights do not depend on the kernel before this one: the first stages start
    // streaming while that kernel is still producing the activations
    const uint32_t ahead = min(kcn, p.stages);
    for (uint32_t i = 0; i < ahead; ++i) load_weights(i);
    pdl_wait();
    for (uint32_t i = 0; i < ahead; ++i) load_activations(i);
    for (uint32_t i = ahead; i < kcn; ++i) {
      const uint32_t s = i % p.stages, round = i / p.stages;
      if (!mbar_wait(&empty_bar[s], (round - 1U) & 1U, abort_flag)) break;
      load_weights(i);
      load_activations(i);
    }
  } else if (tid == 32U) {
    // ---- tensor-core driver
    const uint32_t idesc = (1U << 7U) | (1U << 10U) | ((n_rows >> 3U) << 17U) | ((kTileRows >> 4U) << 24U);
    for (uint32_t i = 0; i < kcn; ++i) {
      const uint32_t s = i % p.stages, round = i / p.stages;
      if (!mbar_wait(&full_bar[s], round & 1U, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t st = smem_u32(smem + static_cast<size_t>(s) * stage_bytes);
      const uint32_t sfa = st + kABytes, b = sfa + kSfBytes, sfb = st + stage_bytes - kSfBytes;
#pragma unroll
      for (uint32_t kb = 0; kb < 4U; ++kb) {
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_sfa + 4U * kb),
                     "l"(umma_desc_sf(sfa + kb * kAtomBytes))
                     : "memory");
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_sfb + 4U * kb),
                     "l"(umma_desc_sf(sfb + kb * kAtomBytes))
                     : "memory");
      }
      uint32_t groups = 4U;
      if constexpr (kPartialK) groups = min(4U, (p.raw >> 1U) - (kc0 + i) * 4U);  // beyond K: zero-filled codes, not issued
#pragma unroll
      for (uint32_t kb = 0; kb < 4U; ++kb) {
        if (kPartialK && kb >= groups) break;
        const uint64_t adesc = umma_desc_sw128(st + kb * 32U);
        const uint64_t bdesc = umma_desc_sw128(b + kb * 32U);
        const uint32_t accumulate = (i > 0U || kb > 0U) ? 1U : 0U;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(tmem_acc), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa + 4U * kb),
            "r"(tmem_sfb + 4U * kb)
            : "memory");
      }
      // the stage may be refilled once these MMAs have read it
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                       smem_u32(&empty_bar[s]))
                   : "memory");
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(&done_bar))
                 : "memory");
  }
  // ---- epilogue: lane = weight row, columns = activation rows
  __syncwarp();
  uint32_t exchange_ranks = 0U, exchange_rank = 0U, exchange_sequence = 0U;
  if constexpr (kExchange) {
    exchange_ranks = e.x.ranks;
    exchange_rank = e.x.rank;
    // The number of this exchange = exchanges produced so far + 1.  Every thread waits for the
    // kernels before this one itself (the counter was advanced by one of them), then reads it
    // while the tensor-core pipeline is still running; the last CTA of this launch stores the
    // new number once every CTA has taken its ticket, i.e. has read the old one.
    pdl_wait();
    exchange_sequence = *reinterpret_cast<const volatile uint32_t*>(e.x.words + 1) + 1U;
  }
  const bool finished = mbar_wait(&done_bar, 0U, abort_flag);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (finished && !*abort_flag) {
    const uint32_t row = blockIdx.x * kTileRows + tid;  // row inside [first_row, first_row + row_count)
    const uint32_t lane_base = tmem_acc + ((warp * 32U) << 16U);
    for (uint32_t c0 = 0; c0 < n_rows; c0 += 16U) {
      uint32_t v[16];
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
            "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
          : "r"(lane_base + c0));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (kExchange) {
        // [rank][split][batch][row_count] in the slot: one 8-byte store {value, sequence} per
        // value and rank, into the peers' memory as well (rank loop outside, so that the
        // accumulator registers keep constant indices)
        if (row < p.row_count) {
          const size_t first = (static_cast<size_t>(exchange_rank) * p.split + blockIdx.y) * p.batch;
          for (uint32_t r = 0; r < exchange_ranks; ++r) {
            uint2* slot = exchange_inbox[r];
#pragma unroll
            for (uint32_t j = 0; j < 16U; ++j) {
              const uint32_t col = n_tile * 128U + c0 + j;
              // one 8-byte store that bypasses L1 (st.global.cg.v2)
              if (col < p.batch) __stcg(slot + (first + col) * p.row_count + row, make_uint2(v[j], exchange_sequence));
            }
          }
        }
      } else if (row < p.row_count) {
#pragma unroll
        for (uint32_t j = 0; j < 16U; ++j) {
          const uint32_t col = n_tile * 128U + c0 + j;
          if (col >= p.batch) continue;
          const float acc = __uint_as_float(v[j]);
          if (p.split == 1U && !(p.raw & 1U))
            p.y[static_cast<size_t>(col) * p.row_count + row] = bf16r(acc * p.weight_scale / p.input_scale);
          else
            p.partials[(static_cast<size_t>(blockIdx.y) * p.batch + col) * p.row_count + row] = acc;
        }
      }
    }
  } else if (tid == 0U && p.error != nullptr) {
    atomicExch(p.error, 100U);  // a pipeline wait ran out: results of this launch are invalid
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0U)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(tmem_cols) : "memory");
  if constexpr (kRopeTail) {
    // every CTA of a tile has stored its partial sums (above); the last one to take the tile's
    // ticket finishes the head.  Release: fence, then ticket; acquire: ticket, then fence.
    __shared__ uint32_t last_of_tile;
    __shared__ __align__(16) float head_rows[8][kTileRows];
    __threadfence();
    __syncthreads();
    if (tid == 0U) {
      const bool last = finished && !*abort_flag && atomicAdd(tail.t.tickets + blockIdx.x, 1U) == p.split - 1U;
      if (last) tail.t.tickets[blockIdx.x] = 0U;   // for the next launch (stream order)
      last_of_tile = last ? 1U : 0U;
    }
    __syncthreads();
    if (last_of_tile) {
      __threadfence();
      const uint32_t row = blockIdx.x * kTileRows + tid;       // output column of the projection
      const size_t stride = static_cast<size_t>(p.batch) * p.row_count;
      for (uint32_t b = 0; b < p.batch; ++b) {
        float sum = 0.0F;
        for (uint32_t sp = 0; sp < p.split; ++sp) sum += __ldcg(p.partials + sp * stride + static_cast<size_t>(b) * p.row_count + row);
        head_rows[b][tid] = bf16r(sum * p.weight_scale / p.input_scale);
      }
      __syncthreads();
      const uint32_t lane = tid & 31U;
      for (uint32_t b = warp; b < p.batch; b += 4U) {
        const float4 v = *reinterpret_cast<const float4*>(&head_rows[b][4U * lane]);
        const float in[4] = {v.x, v.y, v.z, v.w};
        rope_tail_head_row(tail.t, p.first_tile + blockIdx.x, b, in, lane);
      }
    }
  }
  if (kExchange && tid == 0U) {
    // every thread of this CTA has read the sequence number (barrier above); the last CTA of the
    // launch advances it for the kernels that follow in the stream.  The values carry their own
    // sequence word, so nothing here orders them.
    if constexpr (kExchange) {
      const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
      if (atomicAdd(e.x.words + 2, 1U) == total - 1U) {
        e.x.words[2] = 0U;  // for the next launch (stream order)
        e.x.words[1] = exchange_sequence;
      }
    }
  }
}

// Sum of the split-K partials in a fixed order, then the output scale and the BF16 rounding.
__global__ void gemv_mma_finalize_kernel(const float* __restrict__ partials, float* __restrict__ y, uint64_t count,
                                         uint32_t split, float weight_scale, float input_scale) {
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float sum = 0.0F;
  for (uint32_t s = 0; s < split; ++s) sum += partials[static_cast<uint64_t>(s) * count + i];
  y[i] = bf16r(sum * weight_scale / input_scale);
}

int mma_core(const MmaWeights& w, const qllm_matrix& m, uint32_t first_row, uint32_t row_count, uint32_t batch,
             const uint8_t* codes, const uint8_t* atoms, float* partials, float* y, uint32_t* error, bool raw,
             uint32_t* split_out, cudaStream_t stream, const GemvExchange* exchange = nullptr,
             const RopeTail* rope_tail = nullptr);

int launch_gemv_mma(const MmaWeights& w, const qllm_matrix& m, uint32_t first_row, uint32_t row_count,
                    const float* x, float* y, uint32_t batch, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream) {
  if (!w.ready || m.cols % 64U || first_row % kTileRows || !batch || !row_count || row_count > m.rows ||
      first_row > m.rows - row_count || (m.cols % kTileK && batch > 128U))
    return fail(QLLM_INVALID_ARGUMENT, "shape is outside the tensor-core GEMV (K % 64, first row % 128)");
  const uint32_t row_tiles = (row_count + kTileRows - 1U) / kTileRows;
  const uint32_t k_chunks = k_chunks_of(m.cols);
  const uint32_t n_pad = (batch + 15U) / 16U * 16U, n_tiles = (n_pad + 127U) / 128U;
  const uint32_t split = pick_split(row_tiles, n_tiles, k_chunks);
  size_t need = 0;
  const MmaWorkspace ws = carve(workspace, batch, row_count, m.cols, split, &need);
  if (need > workspace_bytes) return fail(QLLM_INVALID_ARGUMENT, "tensor-core GEMV workspace is too small");
  // activations -> packed E2M1 + scale atoms
  const uint64_t items = static_cast<uint64_t>(n_pad) * (m.cols / 16U);
  act_quant_mma_kernel<<<static_cast<unsigned>((items + 127U) / 128U), 128, 0, stream>>>(
      x, ws.codes, ws.atoms, batch, n_pad, m.cols, m.input_scale);
  count_launch();
  int rc = check_launch("act_quant_mma");
  if (rc) return rc;
  rc = mma_core(w, m, first_row, row_count, batch, ws.codes, ws.atoms, ws.partials, y, ws.error, false, nullptr,
                stream);
  if (rc) return rc;
  if (split > 1U) {
    const uint64_t count = static_cast<uint64_t>(batch) * row_count;
    gemv_mma_finalize_kernel<<<static_cast<unsigned>((count + 255U) / 256U), 256, 0, stream>>>(
        ws.partials, y, count, split, m.weight_scale, m.input_scale);
    count_launch();
    rc = check_launch("gemv_mma_finalize");
  }
  return rc;
}

// The tensor-core kernel alone, over the quantised operand that a launch_gemv_mma() call with
// the same workspace, matrix and batch left behind; leaves split-K partials in the workspace.
int launch_gemv_mma_core_only(const MmaWeights& w, const qllm_matrix& m, uint32_t batch, void* workspace,
                              size_t workspace_bytes, cudaStream_t stream) {
  if (!w.ready || m.cols % 64U || !batch || (m.cols % kTileK && batch > 128U))
    return fail(QLLM_INVALID_ARGUMENT, "shape is outside the tensor-core GEMV (K % 64)");
  const uint32_t row_tiles = (m.rows + kTileRows - 1U) / kTileRows;
  const uint32_t n_tiles = ((batch + 15U) / 16U * 16U + 127U) / 128U;  // 128 activation rows per CTA
  const uint32_t split = pick_split(row_tiles, n_tiles, k_chunks_of(m.cols));
  size_t need = 0;
  const MmaWorkspace ws = carve(workspace, batch, m.rows, m.cols, split, &need);
  if (need > workspace_bytes) return fail(QLLM_INVALID_ARGUMENT, "tensor-core GEMV workspace is too small");
  return mma_core(w, m, 0U, m.rows, batch, ws.codes, ws.atoms, ws.partials, nullptr, ws.error, true, nullptr, stream);
}

// Tensor-core GEMV over an operand that is already quantised (codes + atoms).  With `raw`
// the result is left as split-K partials for the consumer; otherwise split == 1 writes y.
int mma_core(const MmaWeights& w, const qllm_matrix& m, uint32_t first_row, uint32_t row_count, uint32_t batch,
             const uint8_t* codes, const uint8_t* atoms, float* partials, float* y, uint32_t* error, bool raw,
             uint32_t* split_out, cudaStream_t stream, const GemvExchange* exchange, const RopeTail* rope_tail) {
  const uint32_t row_tiles = (row_count + kTileRows - 1U) / kTileRows;
  const uint32_t k_chunks = k_chunks_of(m.cols);
  const uint32_t n_pad = (batch + 15U) / 16U * 16U, n_tiles = (n_pad + 127U) / 128U;
  const uint32_t split = pick_split(row_tiles, n_tiles, k_chunks);
  if (split_out) *split_out = split;
  if (exchange && (n_tiles != 1U || static_cast<size_t>(exchange->ranks) * split * batch * row_count >
                                        exchange->capacity))
    return fail(QLLM_INVALID_ARGUMENT, "tensor-parallel exchange slot is too small for this projection");
  MmaWorkspace ws{};
  ws.codes = const_cast<uint8_t*>(codes);
  ws.atoms = const_cast<uint8_t*>(atoms);
  ws.partials = partials;
  ws.error = error;
  int rc = 0;
  CUtensorMap act_map;
  rc = make_codes_map(&act_map, ws.codes, n_pad, m.cols / 2U, std::min(n_pad, 128U));
  if (rc) return rc;
  const uint32_t b_bytes = std::min(n_pad, 128U) * 128U;
  const uint32_t stage_bytes = kABytes + kSfBytes + ((b_bytes + 1023U) & ~1023U) + kSfBytes;
  // as many stages (at most 4) as leave room for two CTAs per SM: the split-K rule above sizes
  // the grid to one wave of two CTAs per SM, whatever the width of the activation tile
  uint32_t stages = 4U;
  while (stages > 2U && stages * stage_bytes > 108U * 1024U) --stages;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 1024U;
  // the opt-in belongs to the device: one entry per device of the process
  static size_t opted_by_device[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  size_t& opted = opted_by_device[device & 63];
  if (smem > opted) {
    rc = check_cuda(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)), "tensor-core GEMV shared memory opt-in");
    if (rc) return rc;
    rc = check_cuda(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)), "tensor-core GEMV shared memory opt-in");
    if (rc) return rc;
    rc = check_cuda(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)), "tensor-core GEMV shared memory opt-in");
    if (rc) return rc;
    rc = check_cuda(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)), "tensor-core GEMV shared memory opt-in");
    if (rc) return rc;
    opted = smem;
  }
  GemvMmaParams p{};
  p.tiled_scales = w.tiled_scales;
  p.act_atoms = ws.atoms;
  p.partials = ws.partials;
  p.y = y;
  p.error = ws.error;
  p.first_tile = first_row / kTileRows;
  p.row_count = row_count;
  p.batch = batch;
  p.n_pad = n_pad;
  p.k_chunks = k_chunks;
  p.k_atoms = padded_atoms(m.cols);
  p.split = split;
  p.stages = stages;
  p.raw = (raw ? 1U : 0U) | ((m.cols / 64U) << 1U);
  p.weight_scale = m.weight_scale;
  p.input_scale = m.input_scale;
  count_launch();
  if (rope_tail != nullptr) {
    if (exchange != nullptr || m.cols % kTileK || first_row != 0U || row_count % kTileRows || batch > 8U || !raw ||
        rope_tail->a.head_dim != kTileRows || rope_tail->a.rotary_dim % 8U ||
        row_count != (rope_tail->a.q_heads + 2U * rope_tail->a.kv_heads) * kTileRows || !rope_tail->tickets)
      return fail(QLLM_INVALID_ARGUMENT, "the fused RoPE / KV-store tail needs head_dim 128, whole heads and at most 8 rows");
    return check_cuda(launch_pdl(nvfp4_gemv_mma_kernel<false, false, true>, dim3(row_tiles, split, n_tiles), dim3(128), smem,
                                 stream, w.codes_map, act_map, p, ExchangeParam<false>{}, TailParam<true>{*rope_tail}),
                      "nvfp4_gemv_mma");
  }
  if (exchange != nullptr)
    return check_cuda(launch_pdl(nvfp4_gemv_mma_kernel<true, true, false>, dim3(row_tiles, split, n_tiles), dim3(128), smem, stream,
                                 w.codes_map, act_map, p, ExchangeParam<true>{*exchange}, TailParam<false>{}), "nvfp4_gemv_mma");
  if (m.cols % kTileK)
    return check_cuda(launch_pdl(nvfp4_gemv_mma_kernel<false, true, false>, dim3(row_tiles, split, n_tiles), dim3(128), smem,
                                 stream, w.codes_map, act_map, p, ExchangeParam<false>{}, TailParam<false>{}), "nvfp4_gemv_mma");
  return check_cuda(launch_pdl(nvfp4_gemv_mma_kernel<false, false, false>, dim3(row_tiles, split, n_tiles), dim3(128), smem, stream,
                               w.codes_map, act_map, p, ExchangeParam<false>{}, TailParam<false>{}), "nvfp4_gemv_mma");
}

// ---- operand buffers and the implementation-neutral GEMV core ---------------------------
size_t quant_buffer_bytes(uint32_t max_rows, uint32_t max_cols) {
  const size_t simt = act_quant_bytes(max_rows, max_cols);
  // the atoms of a partial last stage are read (never used) up to the end of that stage
  const size_t mma = align_up(static_cast<size_t>(128U) * (max_cols / 2U), 1024) +
                     align_up(static_cast<size_t>(padded_atoms(max_cols) + 4U) * kAtomBytes, 1024);
  return std::max(simt, mma) + 1024U;
}

QuantSink make_sink(int gemv_impl, void* quant_buffer, uint32_t rows, uint32_t cols, float g) {
  QuantSink s{};
  s.kind = gemv_impl;
  s.cols = cols;
  s.g = g;
  uint8_t* base = static_cast<uint8_t*>(quant_buffer);
  if (gemv_impl == 0) {
    const size_t values = (static_cast<size_t>(rows) * cols + 15U) & ~static_cast<size_t>(15U);
    s.xi8 = reinterpret_cast<int8_t*>(base);
    s.xscale = reinterpret_cast<float*>(base + values);
  } else {
    s.codes = base;
    s.atoms = base + align_up(static_cast<size_t>(128U) * (cols / 2U), 1024);
  }
  return s;
}

bool gemv_rope_tail_supported(int gemv_impl, const MmaWeights& w, const qllm_matrix& m, uint32_t batch, uint32_t head_dim,
                              uint32_t rotary_dim) {
  return gemv_impl == 1 && w.ready && m.cols % kTileK == 0U && m.rows % kTileRows == 0U && batch <= 8U &&
         head_dim == kTileRows && rotary_dim % 8U == 0U;
}

size_t gemv_partial_floats(uint32_t batch, uint32_t rows, uint32_t cols) {
  if (cols % 64U) return static_cast<size_t>(batch) * rows;
  const uint32_t row_tiles = (rows + kTileRows - 1U) / kTileRows;
  return static_cast<size_t>(pick_split(row_tiles, 1U, k_chunks_of(cols))) * batch * rows;
}

int launch_gemv_core(int gemv_impl, const MmaWeights& w, const qllm_matrix& m, uint32_t first_row,
                     uint32_t row_count, uint32_t batch, void* quant_buffer, float* partials,
                     float* final_out, uint32_t* error, GemvOut* out, cudaStream_t stream,
                     const GemvExchange* exchange, const RopeTail* rope_tail) {
  *out = GemvOut{};
  out->n = row_count;
  out->batch = batch;
  out->weight_scale = m.weight_scale;
  out->input_scale = m.input_scale;
  if (gemv_impl == 1 && w.ready && first_row % kTileRows == 0U && batch <= 128U) {
    const QuantSink s = make_sink(1, quant_buffer, batch, m.cols, m.input_scale);
    uint32_t split = 1;
    const int rc = mma_core(w, m, first_row, row_count, batch, s.codes, s.atoms, partials, nullptr, error, true,
                            &split, stream, exchange, rope_tail);
    out->data = partials;
    out->split = split;
    if (exchange) {
      out->data = reinterpret_cast<const float*>(exchange->inbox[exchange->rank]);  // {value, sequence} pairs
      out->split = exchange->ranks * split;
      out->exchange = exchange->words;
    }
    return rc;
  }
  if (exchange) return fail(QLLM_INVALID_ARGUMENT, "the tensor-parallel exchange needs the tensor-core GEMV");
  if (rope_tail) return fail(QLLM_INVALID_ARGUMENT, "the fused RoPE / KV-store tail needs the tensor-core GEMV");
  if (gemv_impl == 1)
    return fail(QLLM_INVALID_ARGUMENT, "shape is outside the tensor-core GEMV (K % 64, first row % 128, rows <= 128)");
  const int rc = launch_gemv_simt(m, first_row, row_count, quant_buffer, batch, final_out, batch, stream);
  out->data = final_out;
  out->split = 0U;
  return rc;
}

}  // namespace qllm
