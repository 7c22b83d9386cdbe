/*
 * TEST INFRASTRUCTURE -- CPU restatement of the Spherical-KV encode / page-build path.
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may call this;
 * the product never does.
 *
 * Follows, in plain C:
 *   _encode_keys_with_codebooks   spherical_kv_pipeline.py:1130-1144
 *   build_page                    pagebuilder.py:8-33
 *   PageHeader.to_tensor          paging.py:20-31
 *   pack_bits                     bitpacking.py:5-29
 *   pointer-table rows            spherical_kv_pipeline.py:1202-1213, pointer_table.py:10-21
 *
 * Arithmetic order, fixed so that results are reproducible bit for bit (the reference's
 * torch ops leave it to the BLAS / vector ISA of the host):
 *   nsq   = fmaf chain over d = 0..g-1 of k_d*k_d from 0,  r = sqrtf(nsq)
 *   sim_c = fmaf chain over d = 0..g-1 of k_d*cb[c][d] from 0  (k not normalised: the
 *           division by r+1e-8 at spherical_kv_pipeline.py:1138 scales all sim_c alike)
 *   theta = first c with the largest sim_c                      (torch.argmax)
 *   scale = max_t |r| ; code = clamp(rint(r / max(scale,1e-8) * 127), -127, 127)
 * Pinned against the reference itself by tests/golden (see tests/golden/make_golden.py).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

/* r [n][G], theta [n][G] from keys [n][G*g] and codebook [G][C][g] */
void sphkv_oracle_encode(const float* k, const float* cb, int n, int G, int g, int C, float* r,
                         int32_t* theta) {
  for (int t = 0; t < n; ++t) {
    for (int gg = 0; gg < G; ++gg) {
      const float* kg = k + (size_t)t * G * g + (size_t)gg * g;
      float nsq = 0.f;
      for (int d = 0; d < g; ++d) nsq = fmaf(kg[d], kg[d], nsq);
      r[(size_t)t * G + gg] = sqrtf(nsq);
      float best = -INFINITY;
      int code = 0;
      for (int c = 0; c < C; ++c) {
        const float* cw = cb + ((size_t)gg * C + c) * g;
        float s = 0.f;
        for (int d = 0; d < g; ++d) s = fmaf(kg[d], cw[d], s);
        if (s > best) {
          best = s;
          code = c;
        }
      }
      theta[(size_t)t * G + gg] = code;
    }
  }
}

/* bitpacking.py:5-29: value i occupies stream bits [i*b, (i+1)*b), bit k -> byte k>>3, bit k&7 */
void sphkv_oracle_pack_bits(const int32_t* values, int n, int bits, uint8_t* out) {
  const size_t nbytes = ((size_t)n * bits + 7) / 8;
  memset(out, 0, nbytes);
  for (int i = 0; i < n; ++i)
    for (int b = 0; b < bits; ++b)
      if ((values[i] >> b) & 1) {
        const size_t k = (size_t)i * bits + b;
        out[k >> 3] = (uint8_t)(out[k >> 3] + (1u << (k & 7)));
      }
}

static uint16_t f32_to_f16_rn(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
  uint32_t m = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0));
  if (e >= 31) return (uint16_t)(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    m |= 0x800000u;
    const int shift = 14 - e;
    uint32_t h = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (h & 1))) ++h;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)e << 10) | (m >> 13);
  const uint32_t rem = m & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return (uint16_t)(sign | h);
}

/* size of a page with `count` tokens */
int sphkv_oracle_page_nbytes(int count, int G, int bits, int radius_fmt) {
  return 8 + 4 * G + (count * G * bits + 7) / 8 + count * G * (radius_fmt == 1 ? 2 : 1);
}

/* pagebuilder.py:8-33 + paging.py:20-31.  radius_fmt 0: int8 codes; 1: f16 radii.
 * Returns the number of bytes written; theta_rel / radius_rel receive the pointer-table
 * offsets relative to the page start. */
int sphkv_oracle_build_page(const float* r, const int32_t* theta, int count, int G, int bits,
                            int tier_id, int radius_fmt, uint8_t* page, int* theta_rel,
                            int* radius_rel) {
  const int hdr = 8 + 4 * G;
  const int th_bytes = (count * G * bits + 7) / 8;
  memset(page, 0, (size_t)hdr);
  page[0] = (uint8_t)(tier_id & 0xFF);
  page[1] = (uint8_t)(count & 0xFF);
  page[2] = (uint8_t)(radius_fmt & 0xFF);
  for (int gg = 0; gg < G; ++gg) {
    float sc = 0.f;
    for (int t = 0; t < count; ++t) sc = fmaxf(sc, fabsf(r[(size_t)t * G + gg]));
    memcpy(page + 8 + 4 * gg, &sc, 4);
  }
  sphkv_oracle_pack_bits(theta, count * G, bits, page + hdr);
  uint8_t* rp = page + hdr + th_bytes;
  for (int t = 0; t < count; ++t)
    for (int gg = 0; gg < G; ++gg) {
      const float rv = r[(size_t)t * G + gg];
      if (radius_fmt == 1) {
        const uint16_t h = f32_to_f16_rn(rv);
        rp[2 * (t * G + gg)] = (uint8_t)(h & 0xFF);
        rp[2 * (t * G + gg) + 1] = (uint8_t)(h >> 8);
      } else {
        float sc;
        memcpy(&sc, page + 8 + 4 * gg, 4);
        const float safe = sc < 1e-8f ? 1e-8f : sc;
        float q = rintf((rv / safe) * 127.0f); /* round half to even, as torch.round */
        q = q < -127.f ? -127.f : (q > 127.f ? 127.f : q);
        rp[t * G + gg] = (uint8_t)(int8_t)(int)q;
      }
    }
  *theta_rel = hdr;
  *radius_rel = hdr + th_bytes;
  return hdr + th_bytes + count * G * (radius_fmt == 1 ? 2 : 1);
}
