/* CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the arithmetic of the fused SwiGLU path of
 * Forge-researchlab/kernel-POCs, used only as the checker by tests/, by
 * __graft_entry__.smoke() and by the cpu_baseline / --impl reference legs of bench.py.
 * Nothing in the product package may call it.
 *
 * The arithmetic of the reference lives in third-party code that is not in the reference
 * tree: ATen (torch, pinned 2.4.1 by the reference's uv.lock:470-471; 2.11.0 in this image)
 * for its PyTorch composite, and Triton-generated code for its kernels.  This file restates
 * the published elementwise formulas with every rounding point of the reference made
 * explicit.  Parity is PINNED: tests/test_oracle_golden.py checks every function here
 * against vectors produced by running the reference's own swiglu()/swiglu_packed() CPU path
 * in the build container (tests/golden/make_golden.py wrote them), on the shapes, seeds and
 * multipliers of the reference's tests/test_swiglu.py:28-113.
 *
 * Three variants of each direction:
 *
 *   *_chain  the reference's rounding chain, i.e. what
 *            torch_swiglu_reference (kernels/swiglu/swiglu.py:179-188) evaluates and what
 *            autograd derives from it; the Triton kernels round at the same points
 *            (swiglu.py:75-82 forward, :102-116 backward):
 *              z    = f32(gate) * gm                         (fp32)
 *              s    = R(silu_f32(z))                         (cast to the I/O dtype, :187)
 *              h    = R( R(s * up) * dm )                    (:188)
 *              d    = R(dh * dm)
 *              dup  = R(d * s)
 *              dg   = R( f32(R(d * up)) * silu'(z) * gm )    silu'(z) = sig*(1 + z*(1 - sig))
 *            R rounds to nearest even into the I/O dtype; in fp32 every R is the identity
 *            and each binary operation rounds to fp32.
 *   *_once   the same closed form evaluated in fp32 throughout and rounded ONCE into the
 *            I/O dtype: the stated target of the CUDA kernels for bf16/fp16.
 *   *_f64    the closed form in double precision on the (exactly representable) inputs:
 *            the truth both are measured against.
 *
 * Build: see oracle/Makefile (-ffp-contract=off keeps every fp32 operation separately
 * rounded, as the formulas above require).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_F32 0
#define ORACLE_F16 1
#define ORACLE_BF16 2

#define EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------ 16-bit codecs */

static inline float bits_to_f32(uint32_t b) {
  float f;
  memcpy(&f, &b, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  return b;
}

static inline float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

static inline uint16_t f32_to_bf16(float f) { /* round to nearest even; NaN stays NaN */
  uint32_t b = f32_to_bits(f);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x0040u);
  b += 0x7fffu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_to_f32(sign);
    /* subnormal: value = man * 2^-24 */
    float v = (float)man * 5.9604644775390625e-08f;
    return sign ? -v : v;
  }
  if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
  return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

static inline uint16_t f32_to_f16(float f) { /* round to nearest even, IEEE binary16 */
  const uint32_t b = f32_to_bits(f);
  const uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
  const uint32_t a = b & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);            /* NaN */
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);           /* >= 65520 -> inf */
  if (a < 0x33000001u) return sign;                                  /* <= 2^-25 -> 0 (ties to even) */
  if (a < 0x38800000u) {                                             /* subnormal result */
    /* value * 2^24 rounded to nearest even integer */
    const float scaled = bits_to_f32(a) * 16777216.0f;               /* exact */
    const float r = nearbyintf(scaled);                              /* default mode: ties to even */
    return (uint16_t)(sign | (uint16_t)r);
  }
  uint32_t m = a - 0x38000000u; /* rebias exponent (127 -> 15) */
  m += 0x0fffu + ((m >> 13) & 1u);
  return (uint16_t)(sign | (uint16_t)(m >> 13));
}

static inline float load_elem(int dtype, const void* p, int64_t i) {
  switch (dtype) {
    case ORACLE_F32: return ((const float*)p)[i];
    case ORACLE_F16: return f16_to_f32(((const uint16_t*)p)[i]);
    default: return bf16_to_f32(((const uint16_t*)p)[i]);
  }
}

/* R(): round an fp32 value into the I/O dtype and hand it back as fp32. */
static inline float round_io(int dtype, float v) {
  switch (dtype) {
    case ORACLE_F32: return v;
    case ORACLE_F16: return f16_to_f32(f32_to_f16(v));
    default: return bf16_to_f32(f32_to_bf16(v));
  }
}

static inline void store_elem(int dtype, void* p, int64_t i, float v) {
  switch (dtype) {
    case ORACLE_F32: ((float*)p)[i] = v; break;
    case ORACLE_F16: ((uint16_t*)p)[i] = f32_to_f16(v); break;
    default: ((uint16_t*)p)[i] = f32_to_bf16(v); break;
  }
}

static int bad_dtype(int dtype) { return dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16; }

/* ------------------------------------------------------------------ fp32 building blocks
 * silu(z) = z / (1 + exp(-z)) and sigmoid(z) = 1 / (1 + exp(-z)): the forms ATen's CPU
 * kernels evaluate.  Both give NaN at z = -inf (-inf/inf), +inf at z = +inf, as the
 * reference's special-value test expects (tests/test_swiglu.py:102-113). */

static inline float silu_f32(float z) { return z / (1.0f + expf(-z)); }
static inline float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }

/* ------------------------------------------------------------------ reference chain */

EXPORT int swiglu_oracle_fwd_chain(int dtype, int64_t n, const void* gate, const void* up, float gm, float dm,
                                   void* out) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float z = load_elem(dtype, gate, i) * gm;          /* gate.float() * gm        swiglu.py:187 */
    const float s = round_io(dtype, silu_f32(z));            /* silu(...).to(dtype)      swiglu.py:187 */
    const float m = round_io(dtype, s * load_elem(dtype, up, i)); /* silu_gate * up      swiglu.py:188 */
    store_elem(dtype, out, i, m * dm);                       /* (...) * down_multiplier  swiglu.py:188 */
  }
  return 0;
}

EXPORT int swiglu_oracle_bwd_chain(int dtype, int64_t n, const void* dout, const void* gate, const void* up, float gm,
                                   float dm, void* dgate, void* dup) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float g = load_elem(dtype, gate, i);
    const float u = load_elem(dtype, up, i);
    const float z = g * gm;
    const float s = round_io(dtype, silu_f32(z));
    const float d = round_io(dtype, load_elem(dtype, dout, i) * dm); /* grad of (m * dm); kernel: swiglu.py:108 */
    const float du = d * s;                                          /* grad of up;        kernel: swiglu.py:110 */
    const float ds = round_io(dtype, d * u);                         /* grad of silu_gate, in the I/O dtype      */
    const float sig = sigmoid_f32(z);
    const float dz = (ds * sig) * (1.0f + z * (1.0f - sig));         /* ATen's order;      kernel: swiglu.py:111 */
    /* Read both inputs before writing: dgate/dup may be the same buffers as gate/up. */
    store_elem(dtype, dgate, i, dz * gm);
    store_elem(dtype, dup, i, du);
  }
  return 0;
}

/* ------------------------------------------------------------------ fp32 throughout, one rounding */

EXPORT int swiglu_oracle_fwd_once(int dtype, int64_t n, const void* gate, const void* up, float gm, float dm,
                                  void* out) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float z = load_elem(dtype, gate, i) * gm;
    store_elem(dtype, out, i, (silu_f32(z) * load_elem(dtype, up, i)) * dm);
  }
  return 0;
}

EXPORT int swiglu_oracle_bwd_once(int dtype, int64_t n, const void* dout, const void* gate, const void* up, float gm,
                                  float dm, void* dgate, void* dup) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float g = load_elem(dtype, gate, i);
    const float u = load_elem(dtype, up, i);
    const float z = g * gm;
    const float d = load_elem(dtype, dout, i) * dm;
    const float sig = sigmoid_f32(z);
    const float du = d * silu_f32(z);
    const float dz = ((d * u) * sig) * (1.0f + z * (1.0f - sig));
    store_elem(dtype, dgate, i, dz * gm);
    store_elem(dtype, dup, i, du);
  }
  return 0;
}

/* ------------------------------------------------------------------ double precision truth */

EXPORT int swiglu_oracle_fwd_f64(int dtype, int64_t n, const void* gate, const void* up, double gm, double dm,
                                 double* out) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const double z = (double)load_elem(dtype, gate, i) * gm;
    out[i] = (z / (1.0 + exp(-z))) * (double)load_elem(dtype, up, i) * dm;
  }
  return 0;
}

/* Also returns |d*u|, the natural scale of dgate (the derivative factor is O(1) and crosses
 * zero near z = -1.278, where a relative error is meaningless). */
EXPORT int swiglu_oracle_bwd_f64(int dtype, int64_t n, const void* dout, const void* gate, const void* up, double gm,
                                 double dm, double* dgate, double* dup, double* dgate_scale) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const double u = (double)load_elem(dtype, up, i);
    const double z = (double)load_elem(dtype, gate, i) * gm;
    const double d = (double)load_elem(dtype, dout, i) * dm;
    const double sig = 1.0 / (1.0 + exp(-z));
    dup[i] = d * (z * sig);
    dgate[i] = d * u * (sig * (1.0 + z * (1.0 - sig))) * gm;
    if (dgate_scale) dgate_scale[i] = fabs(d * u * gm);
  }
  return 0;
}


/* ------------------------------------------------------------------ GeGLU (sibling operator)
 * h = gelu(gate) * up, reference kernels/geglu/geglu.py: torch_geglu_reference (:255-263) is
 * gelu(gate.float(), approximate).to(dtype) * up with the backward by autograd; the Triton kernels
 * (:90-123, :126-182) use the same formulas.  approximate_tanh != 0 selects the tanh form.
 * ATen's expressions (activation and derivative):
 *   tanh:  inner = sqrt(2/pi) * (x + 0.044715 x^3);  gelu = 0.5 x (1 + tanh(inner))
 *          d/dx  = 0.5 (1 + tanh) + 0.5 x (1 - tanh^2) * sqrt(2/pi) (1 + 3*0.044715 x^2)
 *   erf:   cdf = 0.5 (1 + erf(x / sqrt 2));  gelu = x cdf;  d/dx = cdf + x exp(-x^2/2)/sqrt(2 pi)
 * chain = these in fp32 with the reference's rounding points; once = the cancellation-free closed
 * form (sigmoid / erfc) in fp32 rounded once, the kernels' target; f64 = the truth. */

static inline float gelu_chain_f32(float x, int tanh_form) {
  if (tanh_form) {
    const float inner = 0.7978845608028654f * (x + 0.044715f * (x * x * x));
    return 0.5f * x * (1.0f + tanhf(inner));
  }
  return x * (0.5f * (1.0f + erff(x * 0.7071067811865476f)));
}
static inline float gelu_grad_chain_f32(float x, int tanh_form) {
  if (tanh_form) {
    const float x2 = x * x;
    const float inner = 0.7978845608028654f * (x + 0.044715f * (x2 * x));
    const float t = tanhf(inner);
    const float left_derivative = 0.5f * (1.0f + t);
    const float right_derivative = (0.5f * x) * (1.0f - t * t) * (0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x2));
    return left_derivative + right_derivative;
  }
  const float cdf = 0.5f * (1.0f + erff(x * 0.7071067811865476f));
  const float pdf = expf(-0.5f * x * x) * 0.3989422804014327f;
  return cdf + x * pdf;
}
static inline void gelu_once_f32(float x, int tanh_form, float* act, float* grad) {
  if (tanh_form) {
    const float x2 = x * x;
    const float q = x * (1.5957691216057308f + 0.07135481627f * x2);
    const float e = expf(-q);
    const float den = 1.0f + e;
    const float sig = 1.0f / den;
    const float one_minus_sig = e < 1e30f ? e * sig : 1.0f; /* accurate for large x; no inf * 0 */
    *act = x / den;
    *grad = sig * (1.0f + (x * one_minus_sig) * (1.5957691216057308f + 3.0f * 0.07135481627f * x2));
  } else {
    const float cdf = 0.5f * erfcf(-x * 0.7071067811865476f);
    *act = x * cdf;
    *grad = cdf + x * (0.3989422804014327f * expf(-0.5f * x * x));
  }
}
static inline void gelu_f64(double x, int tanh_form, double* act, double* grad) {
  if (tanh_form) {
    const double q = 2.0 * 0.7978845608028654 * (x + 0.044715 * x * x * x);
    const double sig = 1.0 / (1.0 + exp(-q));
    *act = x * sig;
    *grad = sig * (1.0 + x * (1.0 - sig) * 2.0 * 0.7978845608028654 * (1.0 + 3.0 * 0.044715 * x * x));
  } else {
    const double cdf = 0.5 * erfc(-x * 0.7071067811865476);
    *act = x * cdf;
    *grad = cdf + x * 0.3989422804014327 * exp(-0.5 * x * x);
  }
}

EXPORT int geglu_oracle_fwd(int variant_once, int dtype, int tanh_form, int64_t n, const void* gate, const void* up,
                            void* out) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float g = load_elem(dtype, gate, i), u = load_elem(dtype, up, i);
    if (variant_once) {
      float a, d;
      gelu_once_f32(g, tanh_form, &a, &d);
      store_elem(dtype, out, i, a * u);
    } else {
      const float a = round_io(dtype, gelu_chain_f32(g, tanh_form));   /* gelu(...).to(dtype)  geglu.py:262 */
      store_elem(dtype, out, i, a * u);                                /* activated * up       geglu.py:263 */
    }
  }
  return 0;
}

EXPORT int geglu_oracle_bwd(int variant_once, int dtype, int tanh_form, int64_t n, const void* dout, const void* gate,
                            const void* up, void* dgate, void* dup) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float g = load_elem(dtype, gate, i), u = load_elem(dtype, up, i), d = load_elem(dtype, dout, i);
    float dg, du;
    if (variant_once) {
      float a, gr;
      gelu_once_f32(g, tanh_form, &a, &gr);
      du = d * a;
      dg = (d * u) * gr;
    } else {
      const float a = round_io(dtype, gelu_chain_f32(g, tanh_form));
      du = d * a;                                  /* grad of up: dout * activated (in the I/O dtype) */
      const float da = round_io(dtype, d * u);     /* grad of activated, rounded by autograd          */
      dg = da * gelu_grad_chain_f32(g, tanh_form); /* gelu_backward in fp32, then cast                */
    }
    store_elem(dtype, dgate, i, dg);
    store_elem(dtype, dup, i, du);
  }
  return 0;
}

EXPORT int geglu_oracle_f64(int dtype, int tanh_form, int64_t n, const void* dout, const void* gate, const void* up,
                            double* h, double* dgate, double* dup, double* dgate_scale) {
  if (bad_dtype(dtype) || n < 0) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const double g = load_elem(dtype, gate, i), u = load_elem(dtype, up, i), d = load_elem(dtype, dout, i);
    double a, gr;
    gelu_f64(g, tanh_form, &a, &gr);
    h[i] = a * u;
    dup[i] = d * a;
    dgate[i] = d * u * gr;
    dgate_scale[i] = fabs(d * u);
  }
  return 0;
}

/* ------------------------------------------------------------------ codec access for tests */

EXPORT void swiglu_oracle_to_f32(int dtype, int64_t n, const void* in, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = load_elem(dtype, in, i);
}
EXPORT void swiglu_oracle_from_f32(int dtype, int64_t n, const float* in, void* out) {
  for (int64_t i = 0; i < n; ++i) store_elem(dtype, out, i, in[i]);
}
