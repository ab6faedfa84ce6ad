// Element types: of tensors in weight files (all that safetensors names) and of the engine
// (float32, bfloat16, int32).  The first two values are the dtype codes of the kernels' C entry
// points (0 = float32, 1 = bfloat16).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <string>

namespace illm {

enum class DType : int { F32 = 0, BF16 = 1, F16 = 2, F64 = 3, I64 = 4, I32 = 5, I16 = 6, I8 = 7, U8 = 8, BOOL = 9 };

inline size_t dtype_size(DType t) {
    switch (t) {
        case DType::F64: case DType::I64: return 8;
        case DType::F32: case DType::I32: return 4;
        case DType::BF16: case DType::F16: case DType::I16: return 2;
        default: return 1;
    }
}
inline bool dtype_is_float(DType t) { return t == DType::F32 || t == DType::BF16 || t == DType::F16 || t == DType::F64; }
inline const char* dtype_name(DType t) {   // the names of the safetensors container
    switch (t) {
        case DType::F32: return "F32"; case DType::BF16: return "BF16"; case DType::F16: return "F16";
        case DType::F64: return "F64"; case DType::I64: return "I64"; case DType::I32: return "I32";
        case DType::I16: return "I16"; case DType::I8: return "I8"; case DType::U8: return "U8";
        default: return "BOOL";
    }
}
inline bool dtype_from_name(const std::string& s, DType* out) {
    for (int i = 0; i <= 9; i++)
        if (s == dtype_name((DType)i)) { *out = (DType)i; return true; }
    return false;
}
inline const char* dtype_word(DType t) {   // the names of config.json and of the command lines
    switch (t) {
        case DType::F32: return "float32"; case DType::BF16: return "bfloat16"; case DType::F16: return "float16";
        case DType::I32: return "int32"; default: return dtype_name(t);
    }
}

// float32 -> bfloat16, round to nearest even (what the device's conversion does)
inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);   // NaN stays NaN
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float bf16_bits_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {                      // subnormal: normalise
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            u = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | man << 13;
    } else {
        u = sign | (exp + 127 - 15) << 23 | man << 13;
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

}  // namespace illm
