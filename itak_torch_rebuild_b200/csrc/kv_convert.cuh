// f32 -> f16 conversion shared by every kernel that writes cache elements.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace itk {

// IEEE round-to-nearest-even f32 -> f16 with the reference's NaN rule: every
// NaN becomes sign | 0x7e00 (crates/wgpu-compute/src/kernels/k1_q4k_gemv.rs:285-329).
// The hardware conversion already gives RNE for normals and subnormals,
// overflow to infinity and signed zero on underflow; only its NaN payload differs.
__device__ __forceinline__ unsigned short f32_to_f16_bits(float x) {
    const unsigned short h = __half_as_ushort(__float2half_rn(x));
    if (x != x) return static_cast<unsigned short>(((__float_as_uint(x) >> 16) & 0x8000u) | 0x7e00u);
    return h;
}

// Eight consecutive elements as one 16-byte vector; element 2i in the low half of word i
// (crates/wgpu-compute/tests/kv_f16.rs:164-173).
__device__ __forceinline__ uint4 pack8(const float4& a, const float4& b) {
    uint4 r;
    r.x = f32_to_f16_bits(a.x) | (static_cast<uint32_t>(f32_to_f16_bits(a.y)) << 16);
    r.y = f32_to_f16_bits(a.z) | (static_cast<uint32_t>(f32_to_f16_bits(a.w)) << 16);
    r.z = f32_to_f16_bits(b.x) | (static_cast<uint32_t>(f32_to_f16_bits(b.y)) << 16);
    r.w = f32_to_f16_bits(b.z) | (static_cast<uint32_t>(f32_to_f16_bits(b.w)) << 16);
    return r;
}

}  // namespace itk
