/* CPU restatement of the TurboQuant 3-bit KV codec, d = 128.  TEST INFRASTRUCTURE ONLY.
 *
 * Follows the reference's C++ statement of the codec, tests/test_turbo_quant.cpp in the
 * SwiftLM tree (the production encoder lives in a dependency that is not vendored there):
 *   normalised fast Walsh-Hadamard transform                      :14
 *   forward / inverse rotation  S2 . H . S1  and  S1 . H . S2     :15-16
 *   QJL rotation                Q2 . H . Q1                       :17
 *   nearest-centroid index by boundary search                     :18
 *   3-bit pack / unpack (little-endian bit stream)                :19-20
 *   fp16 conversion by truncation (flush denormals, no rounding)  :21-22
 *   V encode/decode                                               :69-75
 *   K encode/decode with residual sign bits                       :85-98
 * Pinned against the reference's own functions compiled into oracle/_ref/libturbo_ref.so
 * (tests/test_turbo_oracle.py).  Constants come from the generated turbo_tables.h.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include "turbo_tables.h"

static inline float sgn(const unsigned int* neg, int i) { return (neg[i >> 5] >> (i & 31)) & 1u ? -1.f : 1.f; }

void turbo_fwht128(float* x) { /* :14 */
  for (int h = 1; h < 128; h *= 2)
    for (int i = 0; i < 128; i += 2 * h)
      for (int j = i; j < i + h; ++j) {
        const float a = x[j], b = x[j + h];
        x[j] = a + b;
        x[j + h] = a - b;
      }
  for (int i = 0; i < 128; ++i) x[i] *= 0.08838834764831845f; /* 1/sqrt(128) */
}
void turbo_rot_fwd(float* x) { /* :15 */
  for (int i = 0; i < 128; ++i) x[i] *= sgn(TURBO_S1_NEG, i);
  turbo_fwht128(x);
  for (int i = 0; i < 128; ++i) x[i] *= sgn(TURBO_S2_NEG, i);
}
void turbo_rot_inv(float* x) { /* :16 */
  for (int i = 0; i < 128; ++i) x[i] *= sgn(TURBO_S2_NEG, i);
  turbo_fwht128(x);
  for (int i = 0; i < 128; ++i) x[i] *= sgn(TURBO_S1_NEG, i);
}
void turbo_qjl_rot(float* x) { /* :17 */
  for (int i = 0; i < 128; ++i) x[i] *= sgn(TURBO_Q1_NEG, i);
  turbo_fwht128(x);
  for (int i = 0; i < 128; ++i) x[i] *= sgn(TURBO_Q2_NEG, i);
}
int turbo_nearest3(float v) { /* :18: index = number of boundaries <= v */
  int idx = 0;
  for (int i = 0; i < 7; ++i) idx += !(v < TURBO_B3[i]);
  return idx;
}
void turbo_pack3(const uint8_t* idx, uint8_t* out) { /* :19, d = 128 -> 48 bytes */
  memset(out, 0, 48);
  for (int i = 0; i < 128; ++i) {
    const int bo = 3 * i, by = bo >> 3, bi = bo & 7;
    const unsigned v = (unsigned)(idx[i] & 7) << bi;
    out[by] |= (uint8_t)v;
    if (bi > 5) out[by + 1] |= (uint8_t)(v >> 8);
  }
}
void turbo_unpack3(const uint8_t* in, uint8_t* idx) { /* :20 */
  for (int i = 0; i < 128; ++i) {
    const int bo = 3 * i, by = bo >> 3, bi = bo & 7;
    unsigned r = in[by];
    if (by + 1 < 48) r |= (unsigned)in[by + 1] << 8;
    idx[i] = (uint8_t)((r >> bi) & 7);
  }
}
uint16_t turbo_to_f16(float f) { /* :21: truncating conversion, denormals flush to signed zero */
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
  const int32_t e = (int32_t)((u >> 23) & 0xFF) - 127 + 15;
  const uint32_t m = u & 0x7FFFFFu;
  if (e <= 0) return s;
  if (e >= 31) return (uint16_t)(s | 0x7C00u);
  return (uint16_t)(s | (uint16_t)(e << 10) | (uint16_t)(m >> 13));
}
float turbo_from_f16(uint16_t h) { /* :22 */
  const uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  uint32_t u;
  if (!e) u = s;
  else if (e == 31) u = s | (0xFFu << 23) | m;
  else u = s | ((e + 127 - 15) << 23) | (m << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* V: L2-normalise, rotate, 3-bit index, pack; store fp16(||x|| / ||centroid vector||) (:69-74). */
void turbo_encode_v(const float* src, uint8_t packed[48], uint16_t* norm16) {
  float buf[128];
  float ns = 0.f;
  for (int i = 0; i < 128; ++i) ns += src[i] * src[i];
  const float gn = sqrtf(ns), inv = gn > 1e-10f ? 1.f / gn : 0.f;
  for (int i = 0; i < 128; ++i) buf[i] = src[i] * inv;
  turbo_rot_fwd(buf);
  uint8_t idx[128];
  float rs = 0.f;
  for (int i = 0; i < 128; ++i) {
    idx[i] = (uint8_t)turbo_nearest3(buf[i]);
    rs += TURBO_C3[idx[i]] * TURBO_C3[idx[i]];
  }
  const float rn2 = sqrtf(rs), cor = rn2 > 1e-10f ? gn / rn2 : gn;
  turbo_pack3(idx, packed);
  *norm16 = turbo_to_f16(cor);
}
void turbo_decode_v(const uint8_t packed[48], uint16_t norm16, float* dst) { /* :74-75 */
  uint8_t idx[128];
  turbo_unpack3(packed, idx);
  for (int i = 0; i < 128; ++i) dst[i] = TURBO_C3[idx[i]];
  turbo_rot_inv(dst);
  const float sc = turbo_from_f16(norm16);
  for (int i = 0; i < 128; ++i) dst[i] *= sc;
}

/* K: normalise, rotate, index; residual = normalised - inverse-rotated centroids; store the
 * sign bits of the QJL-rotated residual, fp16 ||k|| and fp16 ||residual|| (:88-94). */
void turbo_encode_k(const float* src, uint8_t packed[48], uint8_t signs[16], uint16_t* norm16,
                    uint16_t* rnorm16) {
  float nrm[128], rot[128], mr[128], res[128];
  float ns = 0.f;
  for (int i = 0; i < 128; ++i) ns += src[i] * src[i];
  const float nm = sqrtf(ns), inv = nm > 1e-10f ? 1.f / nm : 0.f;
  for (int i = 0; i < 128; ++i) nrm[i] = src[i] * inv;
  memcpy(rot, nrm, sizeof rot);
  turbo_rot_fwd(rot);
  uint8_t idx[128];
  for (int i = 0; i < 128; ++i) idx[i] = (uint8_t)turbo_nearest3(rot[i]);
  for (int i = 0; i < 128; ++i) mr[i] = TURBO_C3[idx[i]];
  turbo_rot_inv(mr);
  float rns = 0.f;
  for (int i = 0; i < 128; ++i) { res[i] = nrm[i] - mr[i]; rns += res[i] * res[i]; }
  const float rnm = sqrtf(rns);
  turbo_qjl_rot(res);
  memset(signs, 0, 16);
  for (int i = 0; i < 128; ++i) if (res[i] >= 0) signs[i >> 3] |= (uint8_t)(1u << (i & 7));
  turbo_pack3(idx, packed);
  *norm16 = turbo_to_f16(nm);
  *rnorm16 = turbo_to_f16(rnm);
}
/* decode: (centroids rotated back + QJL_C/128 * rnorm * qrot(signs)) * ||k||  (:96-98) */
void turbo_decode_k(const uint8_t packed[48], const uint8_t signs[16], uint16_t norm16,
                    uint16_t rnorm16, float* dst) {
  uint8_t idx[128];
  float sf[128];
  turbo_unpack3(packed, idx);
  for (int i = 0; i < 128; ++i) dst[i] = TURBO_C3[idx[i]];
  turbo_rot_inv(dst);
  for (int i = 0; i < 128; ++i) sf[i] = (signs[i >> 3] & (1u << (i & 7))) ? 1.f : -1.f;
  turbo_qjl_rot(sf);
  const float qs = TURBO_QJL_C / 128.f * turbo_from_f16(rnorm16), sc = turbo_from_f16(norm16);
  for (int i = 0; i < 128; ++i) dst[i] = (dst[i] + sf[i] * qs) * sc;
}
