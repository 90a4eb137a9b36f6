// Device helpers shared by the optimizer kernels: counter-based RNG, dtype-generic vector load/store,
// stochastic rounding to bf16 and the ULP error-correction codec (16-bit float + integer residual).
//
// Numerics follow the PyTorch definitions in heavyball_b200/utils/core.py (parity targets
// heavyball/utils.py:1288-1324 codec, 2341-2370 stochastic rounding).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

// Storage kinds understood by the element-wise kernels.
enum DType : int { kF32 = 0, kBF16 = 1, kF16 = 2, kBF16E8 = 3, kBF16E16 = 4, kF16E8 = 5, kF16E16 = 6, kNone = 7 };

__host__ __device__ inline bool is_ecc(int d) { return d >= kBF16E8 && d <= kF16E16; }
__host__ __device__ inline bool is_bf16_like(int d) { return d == kBF16 || d == kBF16E8 || d == kBF16E16; }
__host__ __device__ inline bool ecc_wide(int d) { return d == kBF16E16 || d == kF16E16; }

// ---------------------------------------------------------------------------------------------
// Philox-4x32-10.  Streams are addressed by (seed, tensor index, element index / 4, draw id), never
// by launch geometry, so results do not depend on grid shape or on which rank runs the update.
// ---------------------------------------------------------------------------------------------
struct Philox {
  uint32_t k0, k1;
  __device__ Philox(uint64_t seed) : k0((uint32_t)seed), k1((uint32_t)(seed >> 32)) {}
  __device__ inline uint4 operator()(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) const {
    uint32_t a = k0, b = k1;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
      uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
      uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
      c0 = hi1 ^ c1 ^ a;
      c1 = lo1;
      c2 = hi0 ^ c3 ^ b;
      c3 = lo0;
      a += 0x9E3779B9u;
      b += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
  }
};

__device__ inline float u32_to_unit(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }  // [0, 1)

// ---------------------------------------------------------------------------------------------
// bf16 stochastic rounding: add 16 uniform low bits, truncate.
// ---------------------------------------------------------------------------------------------
__device__ inline uint16_t sr_bf16_bits(float x, uint32_t rnd16) {
  uint32_t b = __float_as_uint(x);
  b += (rnd16 & 0xFFFFu);
  return (uint16_t)(b >> 16);
}
__device__ inline float bf16_bits_to_float(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }
__device__ inline uint16_t rne_bf16_bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
__device__ inline float f16_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ inline uint16_t rne_f16_bits(float x) { return __half_as_ushort(__float2half_rn(x)); }

// log2(ulp) - 1 of a 16-bit float given its bits.
__device__ inline int half_ulp_log2(uint16_t bits, bool bf16) {
  int m = bf16 ? 7 : 10, bias = bf16 ? 127 : 15;
  int e = (bits & 0x7FFF) >> m;
  return (e == 0 ? 1 - bias - m : e - (bias + m)) - 1;
}

__device__ inline float ecc_decode(uint16_t prim, int corr, bool bf16, float inv_smax) {
  float base = bf16 ? bf16_bits_to_float(prim) : f16_bits_to_float(prim);
  return base + ldexpf((float)corr * inv_smax, half_ulp_log2(prim, bf16));
}

// Returns the residual (integer units) for fp32 value x once prim = RNE(x) is chosen.
__device__ inline int ecc_residual(float x, uint16_t prim, bool bf16, float smax, float unit_rand) {
  float base = bf16 ? bf16_bits_to_float(prim) : f16_bits_to_float(prim);
  float e = ldexpf(x - base, -half_ulp_log2(prim, bf16));
  e = fminf(fmaxf(e, -1.0f), 1.0f) * smax;
  return (int)floorf(e + unit_rand);
}

// ---------------------------------------------------------------------------------------------
// 4-wide generic load / store.  `p` is the primary buffer, `c` the ECC residual buffer (or null).
// ---------------------------------------------------------------------------------------------
struct F4 {
  float v[4];
};

// All loops below have compile-time trip counts and constant indices so that the 4-element
// temporaries live in registers (dynamic indexing would push them to local memory).
__device__ inline void unpack_h4(const void* src, int n_valid, bool fast, uint16_t (&h)[4]) {
  const uint16_t* hp = (const uint16_t*)src;
  if (fast) {
    uint2 t = *(const uint2*)hp;
    h[0] = t.x & 0xFFFF; h[1] = t.x >> 16; h[2] = t.y & 0xFFFF; h[3] = t.y >> 16;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = (k < n_valid) ? hp[k] : (uint16_t)0;
  }
}

__device__ inline F4 load4(const void* p, const void* c, int dt, int64_t i, int n_valid, bool vec_ok) {
  F4 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) r.v[k] = 0.f;
  if (dt == kNone || p == nullptr) return r;
  const bool fast = vec_ok && n_valid == 4;
  if (dt == kF32) {
    const float* f = (const float*)p + i;
    if (fast) {
      float4 t = *(const float4*)f;
      r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < n_valid) r.v[k] = f[k];
    }
    return r;
  }
  uint16_t h[4];
  unpack_h4((const uint16_t*)p + i, n_valid, fast, h);
  const bool bf = is_bf16_like(dt);
  if (!is_ecc(dt)) {
#pragma unroll
    for (int k = 0; k < 4; ++k) r.v[k] = bf ? bf16_bits_to_float(h[k]) : f16_bits_to_float(h[k]);
    return r;
  }
  int corr[4];
  if (ecc_wide(dt)) {
    uint16_t w[4];
    unpack_h4((const uint16_t*)c + i, n_valid, fast, w);
#pragma unroll
    for (int k = 0; k < 4; ++k) corr[k] = (int)(int16_t)w[k];
  } else {
    const int8_t* cp = (const int8_t*)c + i;
    if (fast) {
      uint32_t t = *(const uint32_t*)cp;
#pragma unroll
      for (int k = 0; k < 4; ++k) corr[k] = (int)(int8_t)((t >> (8 * k)) & 0xFF);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) corr[k] = (k < n_valid) ? (int)cp[k] : 0;
    }
  }
  const float inv = ecc_wide(dt) ? (1.0f / 32767.0f) : (1.0f / 127.0f);
#pragma unroll
  for (int k = 0; k < 4; ++k) r.v[k] = ecc_decode(h[k], corr[k], bf, inv);
  return r;
}

__device__ inline void pack_h4(void* dst, int n_valid, bool fast, const uint16_t (&h)[4]) {
  uint16_t* hp = (uint16_t*)dst;
  if (fast) {
    uint2 t;
    t.x = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
    t.y = (uint32_t)h[2] | ((uint32_t)h[3] << 16);
    *(uint2*)hp = t;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < n_valid) hp[k] = h[k];
  }
}

// rnd supplies 4 x 32 random bits: low 16 bits feed bf16 stochastic rounding, the 24 high bits the
// stochastic floor of the ECC residual.
__device__ inline void store4(void* p, void* c, int dt, int64_t i, int n_valid, bool vec_ok, const F4& x, uint4 rnd) {
  if (dt == kNone || p == nullptr) return;
  const bool fast = vec_ok && n_valid == 4;
  const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
  if (dt == kF32) {
    float* f = (float*)p + i;
    if (fast) {
      *(float4*)f = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < n_valid) f[k] = x.v[k];
    }
    return;
  }
  const bool bf = is_bf16_like(dt);
  uint16_t h[4];
  if (!is_ecc(dt)) {
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = bf ? sr_bf16_bits(x.v[k], rr[k]) : rne_f16_bits(x.v[k]);
    pack_h4((uint16_t*)p + i, n_valid, fast, h);
    return;
  }
  int corr[4];
  const float smax = ecc_wide(dt) ? 32767.0f : 127.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    h[k] = bf ? rne_bf16_bits(x.v[k]) : rne_f16_bits(x.v[k]);
    corr[k] = ecc_residual(x.v[k], h[k], bf, smax, u32_to_unit(rr[k]));
  }
  pack_h4((uint16_t*)p + i, n_valid, fast, h);
  if (c == nullptr) return;  // primary-only copy (a peer's replica of a parameter whose residual lives with its owner)
  if (ecc_wide(dt)) {
    uint16_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = (uint16_t)(int16_t)corr[k];
    pack_h4((uint16_t*)c + i, n_valid, fast, w);
  } else {
    int8_t* cp = (int8_t*)c + i;
    if (fast) {
      uint32_t t = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) t |= ((uint32_t)(uint8_t)(int8_t)corr[k]) << (8 * k);
      *(uint32_t*)cp = t;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < n_valid) cp[k] = (int8_t)corr[k];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// NVSwitch multicast accesses (multimem): one instruction acts on the same address of every GPU bound to the
// multicast object.  Addresses must be 16-byte (v4.f32) / 8-byte (v2) aligned.
// ---------------------------------------------------------------------------------------------
__device__ inline F4 mc_ld_reduce4(const void* mc, int dt, int64_t i) {
  F4 r;
  if (dt == kF32) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3])
                 : "l"((const float*)mc + i)
                 : "memory");
  } else {  // four 16-bit values, accumulated in fp32 inside the switch
    uint32_t a, b;
    if (dt == kBF16)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.bf16x2 {%0, %1}, [%2];"
                   : "=r"(a), "=r"(b) : "l"((const uint16_t*)mc + i) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.f16x2 {%0, %1}, [%2];"
                   : "=r"(a), "=r"(b) : "l"((const uint16_t*)mc + i) : "memory");
    const uint16_t h[4] = {(uint16_t)(a & 0xFFFF), (uint16_t)(a >> 16), (uint16_t)(b & 0xFFFF), (uint16_t)(b >> 16)};
#pragma unroll
    for (int k = 0; k < 4; ++k) r.v[k] = dt == kBF16 ? bf16_bits_to_float(h[k]) : f16_bits_to_float(h[k]);
  }
  return r;
}

// Stores the primary of four elements to every GPU through the multicast address `mc`; the residual of an
// error-corrected value (if any) goes to the local buffer `c`.  Same rounding as store4.
__device__ inline void mc_store4(void* mc, void* c, int dt, int64_t i, const F4& x, uint4 rnd) {
  if (dt == kF32) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"((float*)mc + i), "f"(x.v[0]), "f"(x.v[1]), "f"(x.v[2]), "f"(x.v[3])
                 : "memory");
    return;
  }
  const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
  const bool bf = is_bf16_like(dt);
  uint16_t h[4];
  int corr[4] = {0, 0, 0, 0};
  const float smax = ecc_wide(dt) ? 32767.0f : 127.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (is_ecc(dt)) {
      h[k] = bf ? rne_bf16_bits(x.v[k]) : rne_f16_bits(x.v[k]);
      corr[k] = ecc_residual(x.v[k], h[k], bf, smax, u32_to_unit(rr[k]));
    } else {
      h[k] = bf ? sr_bf16_bits(x.v[k], rr[k]) : rne_f16_bits(x.v[k]);
    }
  }
  const float lo = __uint_as_float((uint32_t)h[0] | ((uint32_t)h[1] << 16));
  const float hi = __uint_as_float((uint32_t)h[2] | ((uint32_t)h[3] << 16));
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"((uint16_t*)mc + i), "f"(lo), "f"(hi) : "memory");
  if (is_ecc(dt) && c != nullptr) {
    if (ecc_wide(dt)) {
      uint16_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) w[k] = (uint16_t)(int16_t)corr[k];
      pack_h4((uint16_t*)c + i, 4, true, w);
    } else {
      uint32_t t = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) t |= ((uint32_t)(uint8_t)(int8_t)corr[k]) << (8 * k);
      *(uint32_t*)((int8_t*)c + i) = t;
    }
  }
}

}  // namespace hb
