// Host random streams used for weight init and synthetic batches.
//
// xorshift64 with shifts (13, 7, 17); a uniform draw takes bits [16, 40) of the state as a 24-bit
// fraction; normals are Box-Muller, cosine branch, u1 offset by 1e-7.  This is the recurrence of the
// reference's `RNG` (train/gpt.cu:775-779), so a given seed produces the same weights and tokens.
#include <cmath>
#include <cstdint>

extern "C" {

static inline float u01(uint64_t& st) {
  st ^= st << 13; st ^= st >> 7; st ^= st << 17;
  uint32_t x = (uint32_t)(st >> 16);
  return (float)(x & 0xFFFFFF) / (float)0x1000000;
}

// Fills out[0..n) with scale * N(0,1); returns the advanced state.
uint64_t mlb_rng_normal(uint64_t st, float* out, int64_t n, float scale) {
  for (int64_t i = 0; i < n; i++) {
    float u1 = u01(st) + 1e-7f, u2 = u01(st);
    out[i] = scale * (sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2));
  }
  return st;
}

// out[i] = (int)(u * V), one draw per element.
uint64_t mlb_rng_tokens(uint64_t st, int32_t* out, int64_t n, int32_t V) {
  for (int64_t i = 0; i < n; i++) out[i] = (int32_t)(u01(st) * (float)V);
  return st;
}

// Interleaved draws: ids[i] then tgt[i] (the order the reference's bench modes draw them,
// train/gpt.cu:1390-1392).
uint64_t mlb_rng_token_pairs(uint64_t st, int32_t* ids, int32_t* tgt, int64_t n, int32_t V) {
  for (int64_t i = 0; i < n; i++) {
    ids[i] = (int32_t)(u01(st) * (float)V);
    tgt[i] = (int32_t)(u01(st) * (float)V);
  }
  return st;
}

uint64_t mlb_rng_uniform(uint64_t st, float* out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = u01(st);
  return st;
}

}  // extern "C"
