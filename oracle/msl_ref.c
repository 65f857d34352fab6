/*
 * TEST INFRASTRUCTURE — the CPU oracle for the transformer-forward kernels.
 *
 * A plain-C restatement of the arithmetic of the reference's Metal kernel templates
 * (crates/core/src/kernel_templates.rs), one function per kernel, with the same loop order,
 * the same float accumulation for half types (load -> float, compute, round once on store) and
 * the same corner-case behaviour. Only tests/, __graft_entry__.smoke() and bench.py's CPU
 * baseline may call this; the library never does.
 *
 * Parity pins: every function below is checked in tests/test_oracle_golden.py against the
 * known-answer vectors the reference's own tests hold (tests/golden/known_answers.json lists
 * them with file:line). quantize / dequantize, all bf16 numerics and attention values have no
 * upstream known-answer test: for those, parity is unpinned and rests on this restatement
 * plus PyTorch CPU.
 *
 * Storage type codes: 0 = float32, 1 = float16, 2 = bfloat16.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* ── storage conversions (round-to-nearest-even, as the Metal casts do) ───── */
static float f16_to_f32(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, f;
  if (exp == 0) {
    if (man == 0) f = sign << 31;
    else {
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      man &= 0x3ffu;
      f = (sign << 31) | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) f = (sign << 31) | 0x7f800000u | (man << 13);
  else f = (sign << 31) | ((exp + 112u) << 23) | (man << 13);
  float r; memcpy(&r, &f, 4); return r;
}
static uint16_t f32_to_f16(float v) {
  uint32_t x; memcpy(&x, &v, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xffu) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xffu) == 0xffu) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - exp);
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
  return (uint16_t)(sign | half);
}
static float bf16_to_f32(uint16_t h) { uint32_t f = (uint32_t)h << 16; float r; memcpy(&r, &f, 4); return r; }
static uint16_t f32_to_bf16(float v) {
  uint32_t x; memcpy(&x, &v, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7fffu + lsb;
  return (uint16_t)(x >> 16);
}
static float ld(const void* p, int64_t i, int st) {
  if (st == 0) return ((const float*)p)[i];
  if (st == 1) return f16_to_f32(((const uint16_t*)p)[i]);
  return bf16_to_f32(((const uint16_t*)p)[i]);
}
static void stf(void* p, int64_t i, float v, int st) {
  if (st == 0) ((float*)p)[i] = v;
  else if (st == 1) ((uint16_t*)p)[i] = f32_to_f16(v);
  else ((uint16_t*)p)[i] = f32_to_bf16(v);
}
/* value after one rounding to the storage type */
static float rnd(float v, int st) {
  if (st == 0) return v;
  if (st == 1) return f16_to_f32(f32_to_f16(v));
  return bf16_to_f32(f32_to_bf16(v));
}
API void ref_convert(const void* in, int st_in, void* out, int st_out, int64_t n) {
  for (int64_t i = 0; i < n; i++) stf(out, i, ld(in, i, st_in), st_out);
}

/* matmul{s}: kernel_templates.rs:987-1072. k ascending, float accumulator, batch stride 0 = broadcast. */
API void ref_matmul(const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                    int64_t a_batch_stride, int64_t b_batch_stride, int st) {
  for (int64_t bi = 0; bi < batch; bi++)
    for (int64_t i = 0; i < m; i++)
      for (int64_t j = 0; j < n; j++) {
        float sum = 0.0f;
        for (int64_t kk = 0; kk < k; kk++)
          sum += ld(a, bi * a_batch_stride + i * k + kk, st) * ld(b, bi * b_batch_stride + kk * n + j, st);
        stf(c, (bi * m + i) * n + j, sum, st);
      }
}

/* layer_norm{s}: kernel_templates.rs:1097-1109. Population variance, 1/sqrt(var+eps). */
API void ref_layer_norm(const void* in, const void* gamma, const void* beta, void* out, int64_t rows, int64_t cols, float eps, int st) {
  for (int64_t r = 0; r < rows; r++) {
    int64_t off = r * cols;
    float mean = 0.0f;
    for (int64_t j = 0; j < cols; j++) mean += ld(in, off + j, st);
    mean /= (float)cols;
    float var = 0.0f;
    for (int64_t j = 0; j < cols; j++) { float d = ld(in, off + j, st) - mean; var += d * d; }
    var /= (float)cols;
    float inv_std = 1.0f / sqrtf(var + eps);
    for (int64_t j = 0; j < cols; j++) stf(out, off + j, ld(gamma, j, st) * (ld(in, off + j, st) - mean) * inv_std + ld(beta, j, st), st);
  }
}

/* softmax{s}: kernel_templates.rs:415-421. exp stored in the storage type, then divided. */
API void ref_softmax(const void* in, void* out, int64_t rows, int64_t cols, int st) {
  for (int64_t r = 0; r < rows; r++) {
    int64_t off = r * cols;
    float mx = ld(in, off, st);
    for (int64_t j = 1; j < cols; j++) mx = fmaxf(mx, ld(in, off + j, st));
    float sum = 0.0f;
    for (int64_t j = 0; j < cols; j++) { float e = expf(ld(in, off + j, st) - mx); stf(out, off + j, e, st); sum += e; }
    for (int64_t j = 0; j < cols; j++) stf(out, off + j, ld(out, off + j, st) / sum, st);
  }
}

/* softmax_causal{s}: kernel_templates.rs:478-489. max starts at -1e9; zeros right of the diagonal. */
API void ref_softmax_causal(const void* in, void* out, int64_t batch, int64_t rows, int64_t cols, int st) {
  for (int64_t b = 0; b < batch; b++)
    for (int64_t r = 0; r < rows; r++) {
      int64_t off = (b * rows + r) * cols;
      float mx = -1e9f;
      for (int64_t j = 0; j <= r && j < cols; j++) mx = fmaxf(mx, ld(in, off + j, st));
      float sum = 0.0f;
      for (int64_t j = 0; j < cols; j++) {
        if (j <= r) { float e = expf(ld(in, off + j, st) - mx); stf(out, off + j, e, st); sum += e; }
        else stf(out, off + j, 0.0f, st);
      }
      for (int64_t j = 0; j <= r && j < cols; j++) stf(out, off + j, ld(out, off + j, st) / sum, st);
    }
}

/* gelu{s}: kernel_templates.rs:299-302. tanh form with inner clamped to [-10, 10]. */
API void ref_gelu(const void* in, void* out, int64_t n, int st) {
  for (int64_t i = 0; i < n; i++) {
    float x = ld(in, i, st);
    float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
    inner = fminf(fmaxf(inner, -10.0f), 10.0f);
    stf(out, i, x * 0.5f * (1.0f + tanhf(inner)), st);
  }
}

/* erf_approx + gelu_exact{s}: kernel_templates.rs:312-323, :332. Abramowitz-Stegun 7.1.26. */
static float erf_approx(float x) {
  float ax = fabsf(x);
  float t = 1.0f / (1.0f + 0.3275911f * ax);
  float t2 = t * t, t3 = t2 * t, t4 = t3 * t, t5 = t4 * t;
  float poly = 0.254829592f * t - 0.284496736f * t2 + 1.421413741f * t3 - 1.453152027f * t4 + 1.061405429f * t5;
  float result = 1.0f - poly * expf(-ax * ax);
  return x >= 0.0f ? result : -result;
}
API void ref_gelu_exact(const void* in, void* out, int64_t n, int st) {
  for (int64_t i = 0; i < n; i++) {
    float x = ld(in, i, st);
    stf(out, i, x * 0.5f * (1.0f + erf_approx(x * 0.70710678118f)), st);
  }
}

/* add_bias{s}: kernel_templates.rs:755-757. ch = (i / channel_stride) % num_channels. */
API void ref_add_bias(const void* in, const void* bias, void* out, int64_t numel, int64_t channel_stride, int64_t num_channels, int st) {
  for (int64_t i = 0; i < numel; i++) {
    int64_t ch = (i / channel_stride) % num_channels;
    stf(out, i, ld(in, i, st) + ld(bias, ch, st), st);
  }
}

/* elementwise_{add,sub,mul,div}{s}: kernel_templates.rs:54-88 (contiguous, same-shape form). op: 0 add 1 sub 2 mul 3 div */
API void ref_binary(const void* a, const void* b, void* out, int64_t n, int op, int st) {
  for (int64_t i = 0; i < n; i++) {
    float x = ld(a, i, st), y = ld(b, i, st), z;
    switch (op) { case 0: z = x + y; break; case 1: z = x - y; break; case 2: z = x * y; break; default: z = x / y; }
    stf(out, i, z, st);
  }
}
API void ref_scalar_mul(const void* in, void* out, int64_t n, float scale, int st) {
  for (int64_t i = 0; i < n; i++) stf(out, i, ld(in, i, st) * scale, st);
}

/* embedding{s}: kernel_templates.rs:1134-1138. out[i,:] = W[idx[i],:]; a byte copy, no bounds check upstream. */
API void ref_embedding(const void* w, const int32_t* idx, void* out, int64_t n_idx, int64_t dim, int64_t elem_size) {
  for (int64_t i = 0; i < n_idx; i++)
    memcpy((char*)out + i * dim * elem_size, (const char*)w + (int64_t)idx[i] * dim * elem_size, (size_t)(dim * elem_size));
}

/* gather_dim{0,1}: kernel_templates.rs:888-892, :911-915; index_select_dim{0,1}: :942-946, :965-969. 4-byte elements. */
API void ref_gather(const uint32_t* in, const int32_t* idx, uint32_t* out, int64_t out_rows, int64_t out_cols, int64_t in_cols, int dim) {
  for (int64_t r = 0; r < out_rows; r++)
    for (int64_t c = 0; c < out_cols; c++) {
      int64_t i = r * out_cols + c;
      out[i] = dim == 0 ? in[(int64_t)idx[i] * in_cols + c] : in[r * in_cols + idx[i]];
    }
}
API void ref_index_select(const uint32_t* in, const int32_t* idx, uint32_t* out, int64_t out_rows, int64_t out_cols, int64_t in_cols, int dim) {
  for (int64_t r = 0; r < out_rows; r++)
    for (int64_t c = 0; c < out_cols; c++)
      out[r * out_cols + c] = dim == 0 ? in[(int64_t)idx[r] * in_cols + c] : in[r * in_cols + idx[c]];
}

/* argmax{s}: kernel_templates.rs:511-513. Strict '>' scan from element 0; int32 result. */
API void ref_argmax(const void* in, int32_t* out, int64_t rows, int64_t cols, int st) {
  for (int64_t r = 0; r < rows; r++) {
    int64_t off = r * cols;
    float mx = ld(in, off, st); int32_t mi = 0;
    for (int64_t j = 1; j < cols; j++) { float v = ld(in, off + j, st); if (v > mx) { mx = v; mi = (int32_t)j; } }
    out[r] = mi;
  }
}

/* quantize{ss}_to{ds}: kernel_templates.rs:2210-2211. round() = half away from zero; IEEE divide. */
API void ref_quantize(const void* in, uint8_t* out, int64_t n, float scale, int32_t zero_point, int to_signed, int st) {
  for (int64_t i = 0; i < n; i++) {
    float val = roundf(ld(in, i, st) / scale) + (float)zero_point;
    if (to_signed) { val = fminf(fmaxf(val, -128.0f), 127.0f); out[i] = (uint8_t)(int8_t)val; }
    else { val = fminf(fmaxf(val, 0.0f), 255.0f); out[i] = (uint8_t)val; }
  }
}
/* dequantize{ss}_to{ds}: kernel_templates.rs:2234. Integer subtract first, then float multiply. */
API void ref_dequantize(const uint8_t* in, void* out, int64_t n, float scale, int32_t zero_point, int from_signed, int st) {
  for (int64_t i = 0; i < n; i++) {
    int q = from_signed ? (int)(int8_t)in[i] : (int)in[i];
    stf(out, i, (float)(q - zero_point) * scale, st);
  }
}

/* attention / attention_causal: ops.rs:1559-1569, :1605-1615 — transpose(K), matmul, scalar_mul by
 * 1/sqrt(d_k) (a float), softmax[_causal], matmul; every op materialises in the storage type.
 * q [bh, tq, d], k [bh, tk, d], v [bh, tk, dv], out [bh, tq, dv]; scratch holds tq*tk floats of storage. */
API void ref_attention(const void* q, const void* k, const void* v, void* out, void* scratch, int64_t bh, int64_t tq, int64_t tk,
                       int64_t d, int64_t dv, int causal, int st) {
  float scale = 1.0f / sqrtf((float)d);
  for (int64_t b = 0; b < bh; b++) {
    for (int64_t i = 0; i < tq; i++)
      for (int64_t j = 0; j < tk; j++) {
        float sum = 0.0f;
        for (int64_t c = 0; c < d; c++) sum += ld(q, (b * tq + i) * d + c, st) * ld(k, (b * tk + j) * d + c, st);
        stf(scratch, i * tk + j, rnd(sum, st) * scale, st);
      }
    if (causal) ref_softmax_causal(scratch, scratch, 1, tq, tk, st);
    else ref_softmax(scratch, scratch, tq, tk, st);
    for (int64_t i = 0; i < tq; i++)
      for (int64_t j = 0; j < dv; j++) {
        float sum = 0.0f;
        for (int64_t c = 0; c < tk; c++) sum += ld(scratch, i * tk + c, st) * ld(v, (b * tk + c) * dv + j, st);
        stf(out, (b * tq + i) * dv + j, sum, st);
      }
  }
}

/* Per-output-channel symmetric int8 (no upstream kernel; the definition used by the int8 config):
 * scale[n] = max|w[n,:]| / 127 (1 for an all-zero row), q = clamp(round_half_away(w / scale), -128, 127). */
API void ref_quantize_rows(const void* w, int8_t* q, float* scales, int64_t rows, int64_t cols, int st) {
  for (int64_t r = 0; r < rows; r++) {
    float m = 0.0f;
    for (int64_t j = 0; j < cols; j++) m = fmaxf(m, fabsf(ld(w, r * cols + j, st)));
    float sc = m > 0.0f ? m / 127.0f : 1.0f;
    scales[r] = sc;
    for (int64_t j = 0; j < cols; j++) {
      float val = roundf(ld(w, r * cols + j, st) / sc);
      val = fminf(fmaxf(val, -128.0f), 127.0f);
      q[r * cols + j] = (int8_t)val;
    }
  }
}
/* y[m,n] = (sum_k x[m,k] * q[n,k]) * scale[n], float accumulate, one rounding on store. */
API void ref_matmul_int8(const void* x, const int8_t* q, const float* scales, void* y, int64_t m, int64_t n, int64_t k, int st) {
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < n; j++) {
      float sum = 0.0f;
      for (int64_t c = 0; c < k; c++) sum += ld(x, i * k + c, st) * (float)q[j * k + c];
      stf(y, i * n + j, sum * scales[j], st);
    }
}
