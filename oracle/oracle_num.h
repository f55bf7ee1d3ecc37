// TEST INFRASTRUCTURE — CPU oracle, number formats and the seeded generator.
//
// Only tests, the smoke check and the benchmark's cpu_baseline / reference arm may
// build or call this file. The product library never includes it; the device code
// carries its own, separately written, implementation of the same specification.
//
// PARITY UNPINNED for the LLM path: the reference (strict-lang/Strict) holds no
// GPT-2/Qwen3 forward pass, no quantiser and no generator, so nothing in its tests pins
// these functions. They follow the written specification below. The element-wise
// float semantics follow Strict.Compiler.Cuda/InstructionsToCuda.cs:101-109 (C `float`
// + - * /), pinned by Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:46-57.
//
// Specification (every operation is IEEE-754 binary32 round-to-nearest-even unless it
// is integer arithmetic; no contraction, no fast-math):
//
//  mix64(z)        z=(z^(z>>30))*0xBF58476D1CE4E5B9; z=(z^(z>>27))*0x94D049BB133111EB; z^(z>>31)
//  key(seed,t)     mix64(mix64(seed + GOLD) ^ (t * 0xD6E8FEB86659FD93)),  GOLD=0x9E3779B97F4A7C15
//  rand64(key,c)   mix64(key + (c+1)*GOLD)
//  normal pair j   r=rand64(key,j); k=((uint32)r>>8)+1 in [1,2^24]; b=(uint32)(r>>32)
//                  ln(u)=spec_log(k)-24 ln2 (see below); rad=sqrt(-2 ln u)
//                  angle=(b>>29)+((b>>5)&0xFFFFFF)/2^24 eighths of a turn (see spec_sincos)
//                  element 2j = rad*cos, element 2j+1 = rad*sin
//  uniform int     ((rand64(key,i)>>32) * range) >> 32
//  E4M3 (OCP FN)   bias 7, 3 mantissa bits, no infinity, max 448, NaN 0x7F; encode = RNE,
//                  saturating to +-448
//  bf16            RNE truncation of binary32
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace oracle {

static const uint64_t GOLD = 0x9E3779B97F4A7C15ull;

static inline uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static inline uint64_t stream_key(uint64_t seed, uint64_t tensor) {
  return mix64(mix64(seed + GOLD) ^ (tensor * 0xD6E8FEB86659FD93ull));
}
static inline uint64_t rand64(uint64_t key, uint64_t ctr) { return mix64(key + (ctr + 1) * GOLD); }

static inline float bits_f(uint32_t b) { float f; std::memcpy(&f, &b, 4); return f; }
static inline uint32_t f_bits(float f) { uint32_t b; std::memcpy(&b, &f, 4); return b; }

// ln(k) for an integer k in [1, 2^24], minus 24 ln 2; atanh series on the mantissa.
static inline float spec_log_u(uint32_t k) {
  float f = (float)k;  // exact
  uint32_t b = f_bits(f);
  int e = (int)(b >> 23) - 127;
  float m = bits_f((b & 0x7FFFFFu) | 0x3F800000u);
  if (m > 1.41421354f) { m = m * 0.5f; e += 1; }
  float t = (m - 1.0f) / (m + 1.0f);
  float t2 = t * t;
  float p = std::fmaf(t2, 0.111111111f, 0.142857143f);
  p = std::fmaf(t2, p, 0.2f);
  p = std::fmaf(t2, p, 0.333333343f);
  p = std::fmaf(t2, p, 1.0f);
  float lnm = (t + t) * p;
  return std::fmaf((float)(e - 24), 0.693147182f, lnm);
}

// cos and sin of (oct + frac/2^24) * pi/4, oct in [0,8), frac in [0,2^24).
static inline void spec_sincos(uint32_t oct, uint32_t frac, float* c_out, float* s_out) {
  uint32_t fr = (oct & 1u) ? (16777216u - frac) : frac;
  float a = ((float)fr * 5.9604644775390625e-08f) * 0.785398185f;
  float z = a * a;
  float ps = std::fmaf(z, 2.75573188e-06f, -1.98412701e-04f);
  ps = std::fmaf(z, ps, 8.33333377e-03f);
  ps = std::fmaf(z, ps, -1.66666672e-01f);
  ps = std::fmaf(z, ps, 1.0f);
  float s = a * ps;
  float pc = std::fmaf(z, -2.75573188e-07f, 2.48015876e-05f);
  pc = std::fmaf(z, pc, -1.38888892e-03f);
  pc = std::fmaf(z, pc, 4.16666679e-02f);
  pc = std::fmaf(z, pc, -0.5f);
  float c = std::fmaf(z, pc, 1.0f);
  float cq = (oct & 1u) ? s : c, sq = (oct & 1u) ? c : s;
  switch (oct >> 1) {
    case 0: *c_out = cq; *s_out = sq; break;
    case 1: *c_out = -sq; *s_out = cq; break;
    case 2: *c_out = -cq; *s_out = -sq; break;
    default: *c_out = sq; *s_out = -cq; break;
  }
}

static inline void normal_pair(uint64_t key, uint64_t j, float* z0, float* z1) {
  uint64_t r = rand64(key, j);
  uint32_t k = ((uint32_t)r >> 8) + 1u;
  uint32_t b = (uint32_t)(r >> 32);
  float lnu = spec_log_u(k);
  float rad = std::sqrt(-2.0f * lnu);
  float c, s;
  spec_sincos(b >> 29, (b >> 5) & 0xFFFFFFu, &c, &s);
  *z0 = rad * c;
  *z1 = rad * s;
}
static inline float normal_at(uint64_t key, uint64_t i) {
  float z0, z1;
  normal_pair(key, i >> 1, &z0, &z1);
  return (i & 1) ? z1 : z0;
}
static inline uint32_t uniform_int(uint64_t key, uint64_t i, uint32_t range) {
  return (uint32_t)(((rand64(key, i) >> 32) * (uint64_t)range) >> 32);
}

// ---- bf16 ----
static inline uint16_t f32_to_bf16(float f) {
  uint32_t b = f_bits(f);
  if ((b & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((b >> 16) | 0x40);
  return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
static inline float bf16_to_f32(uint16_t h) { return bits_f((uint32_t)h << 16); }
static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

// ---- FP8 E4M3 (FN) ----
static inline float e4m3_to_f32(uint8_t v) {
  uint32_t s = v >> 7, e = (v >> 3) & 15, m = v & 7;
  float a;
  if (e == 0) a = (float)m * 0.001953125f;            // m * 2^-9
  else if (e == 15 && m == 7) a = NAN;
  else a = std::ldexp((float)(8 + m), (int)e - 10);   // (1+m/8) * 2^(e-7)
  return s ? -a : a;
}
static inline uint8_t f32_to_e4m3(float f) {
  uint32_t b = f_bits(f);
  uint8_t sign = (uint8_t)((b >> 24) & 0x80);
  uint32_t ab = b & 0x7FFFFFFFu;
  if (ab > 0x7F800000u) return 0x7F | sign;
  float a = bits_f(ab);
  if (a >= 448.0f) return 0x7E | sign;
  if (a < 0.015625f) {  // below the smallest normal: units of 2^-9, RNE
    float q = std::nearbyintf(a * 512.0f);
    return (uint8_t)q | sign;
  }
  uint32_t r = ab + 0x7FFFFu + ((ab >> 20) & 1u);
  int e = (int)(r >> 23) - 127;
  uint32_t m = (r >> 20) & 7u;
  uint32_t enc = ((uint32_t)(e + 7) << 3) | m;
  if (enc > 0x7E) enc = 0x7E;
  return (uint8_t)enc | sign;
}

}  // namespace oracle
