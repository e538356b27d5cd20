// Reader of the reference's persistent expert tier files (host code only; no CUDA calls).
//
// The reference persists every expert projection as one file `L{l}.e{i}.{gate,up,down}.bin`
// (`L{l}.shared.*` for the shared expert, `L{l}.router.bin`, `L{l}.shared_gate.bin`) in one of three
// encodings, recognised by the file's byte length (src/moe/residency.rs:511-551):
//   f32    numel * 4 bytes, little-endian floats
//   bf16   numel * 2 bytes, the high halves of the floats
//   qint8  rows * 4 + numel bytes: `rows` f32 scales, then numel int8 codes (row-major)
//          (src/tensor/disk_tier.rs:168-224)
// These functions hand the bytes over in the form the GPU path consumes (int8 codes + scales as they
// are, bf16 as it is, f32 on request), so a tier written by the reference runs without re-encoding.
#include <cstdio>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace {

long long file_size(const char* path) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return -1;
  if (std::fseek(f, 0, SEEK_END) != 0) {
    std::fclose(f);
    return -1;
  }
  long long n = std::ftell(f);
  std::fclose(f);
  return n;
}

int read_exact(const char* path, long long offset, void* dst, size_t bytes) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return ATENIA_ERR_IO;
  int rc = ATENIA_OK;
  if (std::fseek(f, (long)offset, SEEK_SET) != 0 || std::fread(dst, 1, bytes, f) != bytes) rc = ATENIA_ERR_IO;
  std::fclose(f);
  return rc;
}

}  // namespace

extern "C" {

int atenia_tier_detect_dtype(const char* path, int64_t rows, int64_t cols) {
  if (!path) return ATENIA_ERR_NULL;
  if (rows <= 0 || cols <= 0) return ATENIA_ERR_SHAPE;
  const long long n = file_size(path);
  if (n < 0) return ATENIA_ERR_IO;
  const long long numel = rows * cols;
  if (n == numel * 4) return ATENIA_TIER_F32;
  if (n == numel * 2) return ATENIA_TIER_BF16;
  if (n == rows * 4 + numel) return ATENIA_TIER_QINT8;
  return ATENIA_ERR_TIER_FORMAT;
}

int atenia_tier_read_qint8(const char* path, int64_t rows, int64_t cols, int8_t* q, float* scales) {
  if (!path || !q || !scales) return ATENIA_ERR_NULL;
  int dt = atenia_tier_detect_dtype(path, rows, cols);
  if (dt < 0) return dt;
  if (dt != ATENIA_TIER_QINT8) return ATENIA_ERR_TIER_FORMAT;
  int rc = read_exact(path, 0, scales, (size_t)rows * 4);
  if (rc) return rc;
  return read_exact(path, rows * 4, q, (size_t)(rows * cols));
}

int atenia_tier_read_bf16(const char* path, int64_t rows, int64_t cols, uint16_t* out) {
  if (!path || !out) return ATENIA_ERR_NULL;
  int dt = atenia_tier_detect_dtype(path, rows, cols);
  if (dt < 0) return dt;
  if (dt != ATENIA_TIER_BF16) return ATENIA_ERR_TIER_FORMAT;
  return read_exact(path, 0, out, (size_t)(rows * cols) * 2);
}

// Any encoding to f32, as the reference materialises it: f32 as is, bf16 bits << 16, qint8 as
// (f32)q * scale[row] (src/tensor/disk_tier.rs:203-224, :517-536).
int atenia_tier_read_f32(const char* path, int64_t rows, int64_t cols, float* out) {
  if (!path || !out) return ATENIA_ERR_NULL;
  int dt = atenia_tier_detect_dtype(path, rows, cols);
  if (dt < 0) return dt;
  const size_t numel = (size_t)(rows * cols);
  if (dt == ATENIA_TIER_F32) return read_exact(path, 0, out, numel * 4);
  if (dt == ATENIA_TIER_BF16) {
    std::vector<uint16_t> bits(numel);
    int rc = read_exact(path, 0, bits.data(), numel * 2);
    if (rc) return rc;
    for (size_t i = 0; i < numel; ++i) {
      uint32_t u = (uint32_t)bits[i] << 16;
      std::memcpy(&out[i], &u, 4);
    }
    return ATENIA_OK;
  }
  std::vector<int8_t> q(numel);
  std::vector<float> sc((size_t)rows);
  int rc = atenia_tier_read_qint8(path, rows, cols, q.data(), sc.data());
  if (rc) return rc;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) out[r * cols + c] = (float)q[r * cols + c] * sc[r];
  return ATENIA_OK;
}

}  // extern "C"
