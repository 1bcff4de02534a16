// Torch-free element types, reduction ops and host-side numeric helpers
// (bf16 / fp16 conversion) shared by the CPU collectives, the unit tests and
// the host restatements of the device kernels.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>

namespace mccl {

enum class DType : int { F32 = 0, F64, F16, BF16, I8, I16, I32, I64, U8, BOOL, NUM_DTYPES };
enum class RedOp : int { SUM = 0, AVG, MIN, MAX, PRODUCT, BAND, BOR, BXOR, NUM_OPS };

inline size_t dtype_size(DType t) {
  switch (t) {
    case DType::F64: case DType::I64: return 8;
    case DType::F32: case DType::I32: return 4;
    case DType::F16: case DType::BF16: case DType::I16: return 2;
    default: return 1;
  }
}
inline bool dtype_is_float(DType t) {
  return t == DType::F32 || t == DType::F64 || t == DType::F16 || t == DType::BF16;
}
inline const char* dtype_name(DType t) {
  static const char* n[] = {"f32", "f64", "f16", "bf16", "i8", "i16", "i32", "i64", "u8", "bool"};
  return n[static_cast<int>(t)];
}
inline const char* redop_name(RedOp o) {
  static const char* n[] = {"sum", "avg", "min", "max", "product", "band", "bor", "bxor"};
  return n[static_cast<int>(o)];
}

// fp32 → bf16, round to nearest even; NaN stays NaN (quiet).
inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<uint16_t>(u >> 16);
}
inline float bf16_bits_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// IEEE fp16 ↔ fp32 (round to nearest even, handles subnormals / inf / NaN).
inline float f16_bits_to_f32(uint16_t h) {
  uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      u = sign | ((127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_f16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u | (man >> 13) : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    uint32_t shift = static_cast<uint32_t>(14 - exp);
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

}  // namespace mccl
