// Dense QPack records: the on-disk form of the weights this provider consumes.  Host code only.
//
// A record is a 256-byte little-endian header, then the data section, then (256-byte aligned)
// the scale section, padded to a multiple of 4 KiB (docs/expert-pack-v1.md:20-40; header
// fields compiler/expert_pack/constants.py:72-97; writer compiler/expert_pack/writer.py:206-375).
// qllm_pack_check_dense applies the rules of the reference's validator for one dense tensor of
// the manifest's index (compiler/expert_pack/validate.py:131-318) to the record types this
// provider reads: raw F32 / BF16 / I64 tensors (ABI 0) and native NVFP4 matrices (ABI 5:
// packed E2M1 codes, then E4M3FN block scales, the FP32 weight divisor and the FP32 or BF16
// activation divisor).  qllm_pack_nvfp4_matrix turns such a record into the matrix descriptor
// the provider takes, decoding the two divisors the way the reference's provider does
// (runtime/tools/dense_fp4_provider.cpp:3534-3568: weight scale = 1 / divisor, activation
// scale = divisor).
#include <cmath>
#include <cstring>
#include <string>

#include "../../include/qllm_b200.h"

namespace qllm {
int fail(int code, const std::string& message);  // sets qllm_last_error()
}

namespace {

// ---- SHA-256 (FIPS 180-4) -------------------------------------------------------------------------
constexpr uint32_t kRound[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98,
    0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786,
    0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8,
    0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13,
    0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819,
    0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a,
    0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
    0xc67178f2};

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

struct Sha256 {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  uint8_t block[64];
  size_t filled = 0;
  uint64_t total = 0;

  void compress(const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], k = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = k + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + kRound[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      k = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += k;
  }
  void update(const uint8_t* p, size_t n) {
    total += n;
    while (n) {
      if (filled == 0 && n >= 64) { compress(p); p += 64; n -= 64; continue; }
      const size_t take = n < 64 - filled ? n : 64 - filled;
      std::memcpy(block + filled, p, take);
      filled += take; p += take; n -= take;
      if (filled == 64) { compress(block); filled = 0; }
    }
  }
  void finish(uint8_t out[32]) {
    const uint64_t bits = total * 8U;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (filled != 56) update(&zero, 1);
    uint8_t length[8];
    for (int i = 0; i < 8; ++i) length[i] = static_cast<uint8_t>(bits >> (56 - 8 * i));
    update(length, 8);
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) out[4 * i + j] = static_cast<uint8_t>(h[i] >> (24 - 8 * j));
  }
};

// ---- the 256-byte header ---------------------------------------------------------------------------
constexpr size_t kHeaderBytes = 256, kSectionAlignment = 256, kPackAlignment = 4096;
constexpr size_t kHeaderFields = 8 + 2 + 2 + 8 * 4 + 5 * 8 + 32 + 32;  // 148 bytes are fields, the rest is zero
constexpr uint32_t kRowMajor = 1U << 0, kSymmetric = 1U << 2;

struct Header {
  uint16_t version, header_bytes;
  uint32_t flags, quant_abi, rank, dims[5];
  uint64_t record_bytes, data_offset, data_bytes, scale_offset, scale_bytes;
  uint8_t name_hash[32], payload_hash[32];
};

template <class T>
T little(const uint8_t*& p) {
  T v = 0;
  for (size_t i = 0; i < sizeof(T); ++i) v |= static_cast<T>(static_cast<T>(p[i]) << (8 * i));
  p += sizeof(T);
  return v;
}

int bad(const char* message) { return qllm::fail(QLLM_INVALID_ARGUMENT, message); }

float positive_scalar(const uint8_t* p, bool bf16) {
  uint32_t bits = 0;
  if (bf16) bits = (static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8)) << 16;
  else std::memcpy(&bits, p, 4);
  float value;
  std::memcpy(&value, &bits, 4);
  return value;
}

// The checks of one dense index entry against its record; `h` receives the parsed header.
int check_dense(const uint8_t* pack, size_t pack_bytes, const qllm_pack_entry& e, bool verify_payload, Header& h) {
  if (!e.name) return bad("dense record has no name");
  if (e.stored_bytes < kHeaderBytes) return bad("invalid dense size");
  if (e.offset % kPackAlignment || e.stored_bytes % kPackAlignment) return bad("unaligned dense record");
  if (e.offset > pack_bytes || pack_bytes - e.offset < kHeaderBytes) return bad("short dense header");
  const uint8_t* raw = pack + e.offset;
  for (size_t i = kHeaderFields; i < kHeaderBytes; ++i)
    if (raw[i]) return bad("dense header padding is nonzero");
  const uint8_t* p = raw + 8;
  h.version = little<uint16_t>(p);
  h.header_bytes = little<uint16_t>(p);
  h.flags = little<uint32_t>(p);
  h.quant_abi = little<uint32_t>(p);
  h.rank = little<uint32_t>(p);
  for (uint32_t& d : h.dims) d = little<uint32_t>(p);
  h.record_bytes = little<uint64_t>(p);
  h.data_offset = little<uint64_t>(p);
  h.data_bytes = little<uint64_t>(p);
  h.scale_offset = little<uint64_t>(p);
  h.scale_bytes = little<uint64_t>(p);
  std::memcpy(h.name_hash, p, 32);
  std::memcpy(h.payload_hash, p + 32, 32);
  if (std::memcmp(raw, "EPDENS01", 8) != 0 || h.version != 1U) return bad("unknown dense record ABI");
  if (h.header_bytes != kHeaderBytes) return bad("invalid dense header fields");
  if (h.record_bytes != e.stored_bytes) return bad("dense record/manifest size mismatch");
  if (!(h.flags & kRowMajor)) return bad("dense record is not row-major");
  if (h.rank < 1U || h.rank > 5U) return bad("invalid dense rank");
  if (h.rank < 5U && h.dims[4] != 0U) return bad("invalid dense rank padding");
  if (e.rank != h.rank) return bad("dense shape mismatch");
  for (uint32_t i = 0; i < h.rank; ++i)
    if (e.shape[i] != h.dims[i]) return bad("dense shape mismatch");
  uint8_t name_hash[32];
  qllm_sha256(e.name, std::strlen(e.name), name_hash);
  if (std::memcmp(name_hash, h.name_hash, 32) != 0) return bad("dense name hash mismatch");
  if (e.data_offset != h.data_offset || e.data_bytes != h.data_bytes) return bad("dense data section mismatch");
  if (e.scale_offset != h.scale_offset || e.scale_bytes != h.scale_bytes) return bad("dense scale section mismatch");
  if (h.data_offset < kHeaderBytes || h.data_offset > h.record_bytes || h.data_bytes > h.record_bytes - h.data_offset)
    return bad("bad dense data span");
  if (pack_bytes - e.offset < h.record_bytes) return bad("short record read");
  uint64_t elements = 1;
  for (uint32_t i = 0; i < h.rank; ++i) elements *= h.dims[i];
  if (h.quant_abi == 5U) {
    if (!(h.flags & kSymmetric)) return bad("NVFP4 dense flags are incomplete");
    if (h.rank != 2U) return bad("NVFP4 dense storage requires a matrix");
    const uint64_t rows = h.dims[0], columns = h.dims[1];
    if (columns % 16U) return bad("NVFP4 dense columns are not block-aligned");
    const uint64_t local = rows * columns / 16U;
    if (h.data_bytes != rows * columns / 2U) return bad("NVFP4 dense data byte count mismatch");
    if (h.scale_offset % kSectionAlignment) return bad("unaligned NVFP4 dense scales");
    if (h.scale_bytes != local + 6U && h.scale_bytes != local + 8U) return bad("NVFP4 dense scale byte count mismatch");
    if (h.scale_offset > h.record_bytes || h.scale_bytes > h.record_bytes - h.scale_offset)
      return bad("short dense E4M3FN scale read");
    const uint8_t* scales = raw + h.scale_offset;
    for (uint64_t i = 0; i < local; ++i)
      if ((scales[i] & 0x7fU) == 0x7fU) return bad("non-finite dense E4M3FN scale");
    const float weight = positive_scalar(scales + local, false);
    if (!std::isfinite(weight) || !(weight > 0.0F)) return bad("invalid weight global scale");
    const float input = positive_scalar(scales + local + 4U, h.scale_bytes == local + 6U);
    if (!std::isfinite(input) || !(input > 0.0F)) return bad("invalid input global scale");
  } else if (h.quant_abi == 0U) {
    if (h.scale_offset != 0U || h.scale_bytes != 0U) return bad("unknown dense quant ABI");
    if (e.stored_dtype != QLLM_PACK_F32 && e.stored_dtype != QLLM_PACK_BF16 && e.stored_dtype != QLLM_PACK_I64)
      return bad("unknown raw dense dtype");
    const uint64_t width = e.stored_dtype == QLLM_PACK_I64 ? 8U : e.stored_dtype == QLLM_PACK_BF16 ? 2U : 4U;
    if (h.data_bytes != elements * width) return bad("raw dense data byte count mismatch");
  } else {
    return bad("dense quantization ABI is not read by this provider");
  }
  if (verify_payload) {
    uint8_t digest[32];
    qllm_sha256(raw + kHeaderBytes, h.record_bytes - kHeaderBytes, digest);
    if (std::memcmp(digest, h.payload_hash, 32) != 0) return bad("dense payload/header checksum mismatch");
    if (std::memcmp(digest, e.payload_sha256, 32) != 0) return bad("dense payload/manifest checksum mismatch");
  }
  return QLLM_OK;
}

// ---- routed-expert records (EPEXPR01), native NVFP4 ----------------------------------------------
// Header: magic, version, header bytes, flags, quant ABI, layer, expert, hidden, intermediate,
// rows of the first section, reserved, record bytes, four (offset, bytes) pairs — gate+up codes,
// gate+up sidecars, down codes, down sidecars — and the payload SHA-256
// (compiler/expert_pack/constants.py:88-92, writer.py:417-552).  A native NVFP4 matrix's sidecars are its
// E4M3FN block scales, the FP32 weight divisor and the FP32 activation divisor; the first section
// holds gate then up.  Rules of validate_expert_record (validate.py:328-482) for ABI 5.
constexpr uint32_t kGateUpFused = 1U << 1;

struct ExpertHeader {
  uint32_t flags, quant_abi, hidden, intermediate, fused_rows, reserved;
  int32_t layer, expert;
  uint64_t record_bytes, offset[4], bytes[4];
  uint8_t payload_hash[32];
};

int check_expert(const uint8_t* pack, size_t pack_bytes, const qllm_pack_expert_entry& e, bool verify_payload,
                 ExpertHeader& h) {
  if (e.stored_bytes < kHeaderBytes) return bad("invalid expert size");
  if (e.offset % kPackAlignment || e.stored_bytes % kPackAlignment) return bad("unaligned expert record");
  if (e.offset > pack_bytes || pack_bytes - e.offset < kHeaderBytes) return bad("short expert header");
  const uint8_t* raw = pack + e.offset;
  for (size_t i = kHeaderFields; i < kHeaderBytes; ++i)
    if (raw[i]) return bad("expert header padding is nonzero");
  const uint8_t* p = raw + 8;
  const uint16_t version = little<uint16_t>(p), header_bytes = little<uint16_t>(p);
  h.flags = little<uint32_t>(p);
  h.quant_abi = little<uint32_t>(p);
  h.layer = static_cast<int32_t>(little<uint32_t>(p));
  h.expert = static_cast<int32_t>(little<uint32_t>(p));
  h.hidden = little<uint32_t>(p);
  h.intermediate = little<uint32_t>(p);
  h.fused_rows = little<uint32_t>(p);
  h.reserved = little<uint32_t>(p);
  h.record_bytes = little<uint64_t>(p);
  for (int i = 0; i < 4; ++i) {
    h.offset[i] = little<uint64_t>(p);
    h.bytes[i] = little<uint64_t>(p);
  }
  std::memcpy(h.payload_hash, p, 32);
  if (std::memcmp(raw, "EPEXPR01", 8) != 0 || version != 1U) return bad("unknown expert record ABI");
  if (header_bytes != kHeaderBytes || h.reserved != 0U) return bad("invalid expert header fields");
  if (h.quant_abi != 5U) {
    // INT8 (1), FP4 block-32 (3) and its ReLU2 layout (4) are other providers' encodings
    if (h.quant_abi == 1U || h.quant_abi == 3U || h.quant_abi == 4U)
      return bad("expert quantization ABI is not read by this provider");
    return bad("unknown expert quant/layout ABI");
  }
  if (h.flags != (kRowMajor | kSymmetric | kGateUpFused)) return bad("unknown expert quant/layout ABI");
  if (h.layer != e.layer || h.expert != e.expert) return bad("expert identity mismatch");
  if (h.record_bytes != e.stored_bytes) return bad("expert record/manifest size mismatch");
  if (h.fused_rows != 2ULL * h.intermediate) return bad("expert first-section row count mismatch");
  const uint64_t elements = static_cast<uint64_t>(h.hidden) * h.intermediate, local = elements / 16U;
  if (h.hidden % 16U || h.intermediate % 16U) return bad("NVFP4 expert geometry is not block-aligned");
  if (h.bytes[0] != elements) return bad("NVFP4 gate+up byte count mismatch");
  if (h.bytes[1] != 2U * (local + 8U)) return bad("NVFP4 gate+up scale byte count mismatch");
  if (h.bytes[2] != elements / 2U) return bad("NVFP4 down byte count mismatch");
  if (h.bytes[3] != local + 8U) return bad("NVFP4 down scale byte count mismatch");
  for (int i = 0; i < 4; ++i)
    if (e.section_offset[i] != h.offset[i] || e.section_bytes[i] != h.bytes[i]) return bad("expert section index mismatch");
  uint64_t previous_end = kHeaderBytes;
  for (int i = 0; i < 4; ++i) {
    if (h.offset[i] % kSectionAlignment) return bad("unaligned expert section");
    if (h.offset[i] < previous_end) return bad("overlapping expert section");
    if (h.offset[i] > h.record_bytes || h.bytes[i] > h.record_bytes - h.offset[i]) return bad("expert section exceeds record");
    previous_end = h.offset[i] + h.bytes[i];
  }
  if (pack_bytes - e.offset < h.record_bytes) return bad("short record read");
  const uint64_t sidecars[3] = {h.offset[1], h.offset[1] + local + 8U, h.offset[3]};
  static const char* const kNonFinite[3] = {"non-finite gate E4M3FN scale", "non-finite up E4M3FN scale",
                                            "non-finite down E4M3FN scale"};
  static const char* const kWeight[3] = {"invalid gate weight global scale", "invalid up weight global scale",
                                         "invalid down weight global scale"};
  static const char* const kInput[3] = {"invalid gate input global scale", "invalid up input global scale",
                                        "invalid down input global scale"};
  for (int m = 0; m < 3; ++m) {
    const uint8_t* scales = raw + sidecars[m];
    for (uint64_t i = 0; i < local; ++i)
      if ((scales[i] & 0x7fU) == 0x7fU) return bad(kNonFinite[m]);
    const float weight = positive_scalar(scales + local, false), input = positive_scalar(scales + local + 4U, false);
    if (!std::isfinite(weight) || !(weight > 0.0F)) return bad(kWeight[m]);
    if (!std::isfinite(input) || !(input > 0.0F)) return bad(kInput[m]);
  }
  if (e.decoded_bytes != 3U * elements * 4U) return bad("expert decoded byte mismatch");
  if (verify_payload) {
    uint8_t digest[32];
    qllm_sha256(raw + kHeaderBytes, h.record_bytes - kHeaderBytes, digest);
    if (std::memcmp(digest, h.payload_hash, 32) != 0) return bad("expert payload/header checksum mismatch");
    if (std::memcmp(digest, e.payload_sha256, 32) != 0) return bad("expert payload/manifest checksum mismatch");
  }
  return QLLM_OK;
}

}  // namespace

extern "C" {

int qllm_pack_check_expert(const void* pack, size_t pack_bytes, const qllm_pack_expert_entry* entry,
                           int verify_payload) {
  if (!pack || !entry) return bad("null pack or entry");
  ExpertHeader h{};
  return check_expert(static_cast<const uint8_t*>(pack), pack_bytes, *entry, verify_payload != 0, h);
}

int qllm_pack_nvfp4_expert(const void* pack, size_t pack_bytes, const qllm_pack_expert_entry* entry, int verify_payload,
                           qllm_matrix* gate, qllm_matrix* up, qllm_matrix* down) {
  if (!pack || !entry || !gate || !up || !down) return bad("null pack, entry or matrix");
  ExpertHeader h{};
  const int rc = check_expert(static_cast<const uint8_t*>(pack), pack_bytes, *entry, verify_payload != 0, h);
  if (rc) return rc;
  const uint8_t* record = static_cast<const uint8_t*>(pack) + entry->offset;
  const uint64_t elements = static_cast<uint64_t>(h.hidden) * h.intermediate, local = elements / 16U;
  const auto fill = [&](qllm_matrix* m, const uint8_t* codes, const uint8_t* sidecar, uint32_t rows, uint32_t cols) {
    m->codes = codes;
    m->scales = sidecar;
    m->weight_scale = 1.0F / positive_scalar(sidecar + local, false);
    m->input_scale = positive_scalar(sidecar + local + 4U, false);
    m->rows = rows;
    m->cols = cols;
  };
  fill(gate, record + h.offset[0], record + h.offset[1], h.intermediate, h.hidden);
  fill(up, record + h.offset[0] + elements / 2U, record + h.offset[1] + local + 8U, h.intermediate, h.hidden);
  fill(down, record + h.offset[2], record + h.offset[3], h.hidden, h.intermediate);
  return QLLM_OK;
}

void qllm_sha256(const void* bytes, size_t count, uint8_t digest[32]) {
  Sha256 s;
  s.update(static_cast<const uint8_t*>(bytes), count);
  s.finish(digest);
}

int qllm_pack_check_dense(const void* pack, size_t pack_bytes, const qllm_pack_entry* entry, int verify_payload) {
  if (!pack || !entry) return bad("null pack or entry");
  Header h{};
  return check_dense(static_cast<const uint8_t*>(pack), pack_bytes, *entry, verify_payload != 0, h);
}

int qllm_pack_nvfp4_matrix(const void* pack, size_t pack_bytes, const qllm_pack_entry* entry, int verify_payload,
                           qllm_matrix* matrix) {
  if (!pack || !entry || !matrix) return bad("null pack, entry or matrix");
  Header h{};
  const int rc = check_dense(static_cast<const uint8_t*>(pack), pack_bytes, *entry, verify_payload != 0, h);
  if (rc) return rc;
  if (h.quant_abi != 5U) return bad("FP4 tensor has the wrong quantization ABI");
  const uint8_t* record = static_cast<const uint8_t*>(pack) + entry->offset;
  const uint64_t local = static_cast<uint64_t>(h.dims[0]) * h.dims[1] / 16U;
  const uint8_t* scales = record + h.scale_offset;
  matrix->codes = record + h.data_offset;
  matrix->scales = scales;
  matrix->weight_scale = 1.0F / positive_scalar(scales + local, false);
  matrix->input_scale = positive_scalar(scales + local + 4U, h.scale_bytes == local + 6U);
  matrix->rows = h.dims[0];
  matrix->cols = h.dims[1];
  return QLLM_OK;
}

}  // extern "C"
