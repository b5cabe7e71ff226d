// SwiGLU activation kernels for sm_100a (B200).
//
// Replaces the four Triton kernels of the reference
// (kernels/swiglu/swiglu.py:60-176: _swiglu_forward_kernel, _swiglu_backward_kernel and
// their packed twins).  The reference gives one program per token row and pads the row
// to the next power of two; here the problem is a flat stream of 16- or 32-byte vectors
// walked grid-stride by a fixed-size grid, so no lane is masked except in the last tile
// and the row width is unlimited (64-bit indexing).
//
// Numerics (I/O dtype T, all arithmetic in fp32 registers):
//   z = f32(gate) * gm          sigma = 1 / (1 + exp(-z))        silu = z * sigma
//   forward   h     = R( silu * f32(up) * dm )
//   backward  d     = f32(dh) * dm
//             dup   = R( d * silu )
//             dgate = R( d * f32(up) * sigma * (1 + z * (1 - sigma)) * gm )
// R rounds once, to nearest even, into T.  For fp32 I/O the operation order follows the
// ATen composite the reference tests compare with (swiglu.py:179-188 and the autograd
// graph it builds), exp and the division are the accurate ones; for bf16/fp16 I/O the
// exponential is ex2.approx and the reciprocal rcp.approx, the multipliers are folded into
// per-launch constants, and the error (~1e-6 relative) is far below half an ulp of a 16-bit
// result.
//
// Memory: every kernel is a pure stream.  Algorithmic traffic per element of size s is
// 3*s bytes forward (read gate, up; write h) and 5*s backward (read dh, gate, up; write
// dgate, dup).  Nothing is re-read, so loads bypass L1 allocation and stores are
// streaming.  dgate/dup may alias gate/up exactly (the reference's default in-place
// backward, swiglu.py:247-248, 310): each thread loads all of a tile's vectors before
// it stores any, and aliased inputs are never read through the non-coherent path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace swiglu_b200 {

// ---------------------------------------------------------------------------------------
// Vector register blocks and global-memory access with explicit cache behaviour.
// ---------------------------------------------------------------------------------------

enum LdMode : int {
  LD_PLAIN = 0,      // ld.global                        (coherent; safe when outputs alias inputs)
  LD_NC_NOALLOC = 1, // ld.global.nc.L1::no_allocate     (read-only data, never written by this launch)
  LD_CS = 2,         // ld.global.cs                     (coherent, evict-first)
  LD_NC_EF = 3,      // 32-byte only: .nc + L1::no_allocate + L2::evict_first
};
enum StMode : int {
  ST_PLAIN = 0,      // st.global
  ST_CS = 1,         // st.global.cs                     (streaming)
  ST_NOALLOC = 2,    // st.global.L1::no_allocate
  ST_EF = 3,         // 32-byte only: L1::no_allocate + L2::evict_first
};

template <int BYTES> struct Vec;  // BYTES of payload held in 32-bit registers (16-bit for BYTES == 2)
template <> struct Vec<32> { uint32_t w[8]; };
template <> struct Vec<16> { uint32_t w[4]; };
template <> struct Vec<8>  { uint32_t w[2]; };
template <> struct Vec<4>  { uint32_t w[1]; };
template <> struct Vec<2>  { uint32_t w[1]; };  // low 16 bits used

template <int BYTES, int MODE> struct Ld;
template <int BYTES, int MODE> struct St;

#define SWIGLU_LD32(MODE, QUAL)                                                                   \
  template <> struct Ld<32, MODE> {                                                               \
    static __device__ __forceinline__ Vec<32> ld(const void* p) {                                 \
      Vec<32> v;                                                                                  \
      asm volatile("ld.global" QUAL ".v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"                    \
                   : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]),        \
                     "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])                                     \
                   : "l"(p) : "memory");                                                          \
      return v;                                                                                   \
    }                                                                                             \
  };
#define SWIGLU_LD16(MODE, QUAL)                                                                   \
  template <> struct Ld<16, MODE> {                                                               \
    static __device__ __forceinline__ Vec<16> ld(const void* p) {                                 \
      Vec<16> v;                                                                                  \
      asm volatile("ld.global" QUAL ".v4.u32 {%0,%1,%2,%3}, [%4];"                                \
                   : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])                       \
                   : "l"(p) : "memory");                                                          \
      return v;                                                                                   \
    }                                                                                             \
  };
#define SWIGLU_LD8(MODE, QUAL)                                                                    \
  template <> struct Ld<8, MODE> {                                                                \
    static __device__ __forceinline__ Vec<8> ld(const void* p) {                                  \
      Vec<8> v;                                                                                   \
      asm volatile("ld.global" QUAL ".v2.u32 {%0,%1}, [%2];"                                      \
                   : "=r"(v.w[0]), "=r"(v.w[1]) : "l"(p) : "memory");                             \
      return v;                                                                                   \
    }                                                                                             \
  };
#define SWIGLU_LD4(MODE, QUAL)                                                                    \
  template <> struct Ld<4, MODE> {                                                                \
    static __device__ __forceinline__ Vec<4> ld(const void* p) {                                  \
      Vec<4> v;                                                                                   \
      asm volatile("ld.global" QUAL ".u32 %0, [%1];" : "=r"(v.w[0]) : "l"(p) : "memory");         \
      return v;                                                                                   \
    }                                                                                             \
  };
#define SWIGLU_LD2(MODE, QUAL)                                                                    \
  template <> struct Ld<2, MODE> {                                                                \
    static __device__ __forceinline__ Vec<2> ld(const void* p) {                                  \
      uint16_t h;                                                                                 \
      asm volatile("ld.global" QUAL ".u16 %0, [%1];" : "=h"(h) : "l"(p) : "memory");              \
      Vec<2> v;                                                                                   \
      v.w[0] = h;                                                                                 \
      return v;                                                                                   \
    }                                                                                             \
  };
#define SWIGLU_LD_ALL(MODE, QUAL) \
  SWIGLU_LD32(MODE, QUAL) SWIGLU_LD16(MODE, QUAL) SWIGLU_LD8(MODE, QUAL) SWIGLU_LD4(MODE, QUAL) SWIGLU_LD2(MODE, QUAL)

SWIGLU_LD_ALL(LD_PLAIN, "")
SWIGLU_LD_ALL(LD_NC_NOALLOC, ".nc.L1::no_allocate")
SWIGLU_LD_ALL(LD_CS, ".cs")
SWIGLU_LD32(LD_NC_EF, ".nc.L1::no_allocate.L2::evict_first")
// The L2 eviction qualifier exists for 32-byte accesses only; narrower widths keep the L1 hint.
SWIGLU_LD16(LD_NC_EF, ".nc.L1::no_allocate")
SWIGLU_LD8(LD_NC_EF, ".nc.L1::no_allocate")
SWIGLU_LD4(LD_NC_EF, ".nc.L1::no_allocate")
SWIGLU_LD2(LD_NC_EF, ".nc.L1::no_allocate")

#define SWIGLU_ST32(MODE, QUAL)                                                                   \
  template <> struct St<32, MODE> {                                                               \
    static __device__ __forceinline__ void st(void* p, const Vec<32>& v) {                        \
      asm volatile("st.global" QUAL ".v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"                    \
                   :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]),    \
                      "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7]) : "memory");                          \
    }                                                                                             \
  };
#define SWIGLU_ST16(MODE, QUAL)                                                                   \
  template <> struct St<16, MODE> {                                                               \
    static __device__ __forceinline__ void st(void* p, const Vec<16>& v) {                        \
      asm volatile("st.global" QUAL ".v4.u32 [%0], {%1,%2,%3,%4};"                                \
                   :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");     \
    }                                                                                             \
  };
#define SWIGLU_ST8(MODE, QUAL)                                                                    \
  template <> struct St<8, MODE> {                                                                \
    static __device__ __forceinline__ void st(void* p, const Vec<8>& v) {                         \
      asm volatile("st.global" QUAL ".v2.u32 [%0], {%1,%2};"                                      \
                   :: "l"(p), "r"(v.w[0]), "r"(v.w[1]) : "memory");                               \
    }                                                                                             \
  };
#define SWIGLU_ST4(MODE, QUAL)                                                                    \
  template <> struct St<4, MODE> {                                                                \
    static __device__ __forceinline__ void st(void* p, const Vec<4>& v) {                         \
      asm volatile("st.global" QUAL ".u32 [%0], %1;" :: "l"(p), "r"(v.w[0]) : "memory");          \
    }                                                                                             \
  };
#define SWIGLU_ST2(MODE, QUAL)                                                                    \
  template <> struct St<2, MODE> {                                                                \
    static __device__ __forceinline__ void st(void* p, const Vec<2>& v) {                         \
      asm volatile("st.global" QUAL ".u16 [%0], %1;" :: "l"(p), "h"((uint16_t)v.w[0]) : "memory"); \
    }                                                                                             \
  };
#define SWIGLU_ST_ALL(MODE, QUAL) \
  SWIGLU_ST32(MODE, QUAL) SWIGLU_ST16(MODE, QUAL) SWIGLU_ST8(MODE, QUAL) SWIGLU_ST4(MODE, QUAL) SWIGLU_ST2(MODE, QUAL)

SWIGLU_ST_ALL(ST_PLAIN, "")
SWIGLU_ST_ALL(ST_CS, ".cs")
SWIGLU_ST_ALL(ST_NOALLOC, ".L1::no_allocate")
SWIGLU_ST32(ST_EF, ".L1::no_allocate.L2::evict_first")
SWIGLU_ST16(ST_EF, ".L1::no_allocate")
SWIGLU_ST8(ST_EF, ".L1::no_allocate")
SWIGLU_ST4(ST_EF, ".L1::no_allocate")
SWIGLU_ST2(ST_EF, ".L1::no_allocate")

// ---------------------------------------------------------------------------------------
// Element codecs: BYTES of packed T <-> fp32 registers.
// ---------------------------------------------------------------------------------------

template <class T> struct Codec;

template <> struct Codec<float> {
  static constexpr int kSize = 4;
  template <int BYTES> static __device__ __forceinline__ void unpack(const Vec<BYTES>& v, float* f) {
#pragma unroll
    for (int i = 0; i < BYTES / 4; ++i) f[i] = __uint_as_float(v.w[i]);
  }
  template <int BYTES> static __device__ __forceinline__ void pack(const float* f, Vec<BYTES>& v) {
#pragma unroll
    for (int i = 0; i < BYTES / 4; ++i) v.w[i] = __float_as_uint(f[i]);
  }
};

template <> struct Codec<__nv_bfloat16> {
  static constexpr int kSize = 2;
  template <int BYTES> static __device__ __forceinline__ void unpack(const Vec<BYTES>& v, float* f) {
    if constexpr (BYTES == 2) {
      f[0] = __uint_as_float(v.w[0] << 16);
    } else {
#pragma unroll
      for (int i = 0; i < BYTES / 4; ++i) {
        f[2 * i] = __uint_as_float(v.w[i] << 16);             // bf16 -> fp32 is exact: append 16 zero bits
        f[2 * i + 1] = __uint_as_float(v.w[i] & 0xffff0000u);
      }
    }
  }
  template <int BYTES> static __device__ __forceinline__ void pack(const float* f, Vec<BYTES>& v) {
    if constexpr (BYTES == 2) {
      v.w[0] = __bfloat16_as_ushort(__float2bfloat16_rn(f[0]));
    } else {
#pragma unroll
      for (int i = 0; i < BYTES / 4; ++i) {
        __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);  // one cvt.rn.bf16x2.f32
        v.w[i] = *reinterpret_cast<uint32_t*>(&b);
      }
    }
  }
};

template <> struct Codec<__half> {
  static constexpr int kSize = 2;
  template <int BYTES> static __device__ __forceinline__ void unpack(const Vec<BYTES>& v, float* f) {
    if constexpr (BYTES == 2) {
      f[0] = __half2float(__ushort_as_half((unsigned short)v.w[0]));
    } else {
#pragma unroll
      for (int i = 0; i < BYTES / 4; ++i) {
        uint32_t w = v.w[i];
        float2 p = __half22float2(*reinterpret_cast<__half2*>(&w));
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
      }
    }
  }
  template <int BYTES> static __device__ __forceinline__ void pack(const float* f, Vec<BYTES>& v) {
    if constexpr (BYTES == 2) {
      v.w[0] = __half_as_ushort(__float2half_rn(f[0]));
    } else {
#pragma unroll
      for (int i = 0; i < BYTES / 4; ++i) {
        __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        v.w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
  }
};

// ---------------------------------------------------------------------------------------
// The arithmetic.  FAST selects the approximate transcendental pair used for 16-bit I/O.
// ---------------------------------------------------------------------------------------

enum Activation : int { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_GELU_ERF = 2 };

template <bool FAST, int ACT = ACT_SILU> struct Math;

// Per-launch constants derived from the two multipliers, computed once per thread.
struct Consts {
  float gm, dm;
  float neg_gm_log2e;   // -gm * log2(e):       exp(-z) = ex2(gate * neg_gm_log2e)
  float gm_dm_quarter;  //  gm * dm / 4
  float gm_dm;          //  gm * dm
  __device__ __forceinline__ Consts(float gm_, float dm_)
      : gm(gm_), dm(dm_), neg_gm_log2e(gm_ * -1.4426950408889634f), gm_dm_quarter(gm_ * dm_ * 0.25f),
        gm_dm(gm_ * dm_) {}
};

template <> struct Math<true, ACT_SILU> {
  // sigmoid(z)/... via r = 1 / ((1 + exp(-z)) / 4).  Dividing the denominator by four (folded into
  // one FMA) keeps r a normal number for every finite exp(-z) <= 2^128, so the flush-to-zero
  // reciprocal loses nothing; the factor 1/4 is multiplied back where it is exact.
  static __device__ __forceinline__ float quarter_recip(float g, const Consts& c) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * c.neg_gm_log2e));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(e, 0.25f, 0.25f)));
    return r;  // 4 * sigmoid(g * gm)
  }
  static __device__ __forceinline__ float fwd(float g, float u, const Consts& c) {
    return ((g * c.gm_dm_quarter) * quarter_recip(g, c)) * u;
  }
  static __device__ __forceinline__ void bwd(float dh, float g, float u, const Consts& c, float& dgate, float& dup) {
    const float sig = quarter_recip(g, c) * 0.25f;
    const float z = g * c.gm;
    dup = (dh * c.dm) * (z * sig);
    dgate = ((dh * c.gm_dm) * u) * (sig * fmaf(z, 1.0f - sig, 1.0f));
  }
  // fwd and bwd of the same element off one exponential; each result is the expression above, bit for bit.
  static __device__ __forceinline__ void bwd_h(float dh, float g, float u, const Consts& c, float& h, float& dgate,
                                               float& dup) {
    const float qr = quarter_recip(g, c);
    const float sig = qr * 0.25f;
    const float z = g * c.gm;
    h = ((g * c.gm_dm_quarter) * qr) * u;
    dup = (dh * c.dm) * (z * sig);
    dgate = ((dh * c.gm_dm) * u) * (sig * fmaf(z, 1.0f - sig, 1.0f));
  }
};

// fp32 I/O: 1 / (1 + exp(-z)) by rcp.approx (at most 1 ulp off) and silu as z times that, instead of two IEEE
// divisions: the backward of fp32 [32768, 11008] went from 6.76 to 7.02 TB/s, and every result stays within
// 4e-7 relative of the exact value (the contract is 1e-6).  0 restores the divisions.
#ifndef SWIGLU_F32_RCP
#define SWIGLU_F32_RCP 1
#endif

template <> struct Math<false, ACT_SILU> {
  // Same expression tree as ATen's silu / silu_backward, which is what the reference's
  // torch_swiglu_reference (swiglu.py:179-188) evaluates under autograd.
  // 1 / den for den = 1 + exp(-z) >= 1 (or +inf, or NaN).
  static __device__ __forceinline__ float recip(float den) {
#if SWIGLU_F32_RCP
    float r;
    asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(den));  // at most 1 ulp off; 0 for +inf, NaN for NaN
    return r;
#else
    return 1.0f / den;
#endif
  }
  static __device__ __forceinline__ float fwd(float g, float u, const Consts& c) {
    float z = g * c.gm;
#if SWIGLU_F32_RCP
    float silu = z * recip(1.0f + expf(-z));
#else
    float silu = z / (1.0f + expf(-z));
#endif
    return (silu * u) * c.dm;
  }
  static __device__ __forceinline__ void bwd(float dh, float g, float u, const Consts& c, float& dgate, float& dup) {
    float z = g * c.gm;
    float den = 1.0f + expf(-z);
    float sig = recip(den);
#if SWIGLU_F32_RCP
    float silu = z * sig;
#else
    float silu = z / den;
#endif
    float d = dh * c.dm;
    dup = d * silu;
    dgate = (((d * u) * sig) * (1.0f + z * (1.0f - sig))) * c.gm;
  }
  static __device__ __forceinline__ void bwd_h(float dh, float g, float u, const Consts& c, float& h, float& dgate,
                                               float& dup) {
    float z = g * c.gm;
    float den = 1.0f + expf(-z);
    float sig = recip(den);
#if SWIGLU_F32_RCP
    float silu = z * sig;
#else
    float silu = z / den;
#endif
    float d = dh * c.dm;
    h = (silu * u) * c.dm;
    dup = d * silu;
    dgate = (((d * u) * sig) * (1.0f + z * (1.0f - sig))) * c.gm;
  }
};

// ---------------------------------------------------------------------------------------
// GeGLU (the sibling operator, reference kernels/geglu/geglu.py:90-123): h = gelu(gate) * up with
// the tanh approximation or the exact erf form; no multipliers.
//
// tanh form: 0.5*(1 + tanh(a)) is sigmoid(2a), so gelu_tanh(x) = x * sigmoid(q(x)) with
// q(x) = 2*sqrt(2/pi)*(x + 0.044715 x^3).  Evaluated that way the negative tail keeps its relative
// accuracy (1 + tanh cancels there) and the silu machinery is reused:
//   d/dx = s * (1 + x * (1 - s) * q'(x)),   q'(x) = 2*sqrt(2/pi)*(1 + 3*0.044715 x^2).
// erf form: Phi(x) = 0.5*erfc(-x/sqrt 2) (erfc, not 1+erf, again for the negative tail),
//   gelu = x*Phi,  d/dx = Phi + x*exp(-x^2/2)/sqrt(2 pi).
// ---------------------------------------------------------------------------------------

struct GeluConst {
  static constexpr float kQ1 = 1.5957691216057308f;    // 2*sqrt(2/pi)
  static constexpr float kQ3 = 0.07135481627f;         // 2*sqrt(2/pi)*0.044715
  static constexpr float kLog2e = 1.4426950408889634f;
  static constexpr float kInvSqrt2 = 0.7071067811865476f;
  static constexpr float kInvSqrt2Pi = 0.3989422804014327f;
  static constexpr float kErfcT = 0.28284271247461906f;  // 0.4 / sqrt 2: t = 1 / (1 + 0.4 * |x| / sqrt 2)
};

template <> struct Math<true, ACT_GELU_TANH> {
  // 4*sigmoid(q(x)) by one ex2 and one rcp; see Math<true, ACT_SILU>::quarter_recip.
  static __device__ __forceinline__ float quarter_recip(float x, float x2) {
    float e, r;
    const float t = x * fmaf(x2, -GeluConst::kQ3 * GeluConst::kLog2e, -GeluConst::kQ1 * GeluConst::kLog2e);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(e, 0.25f, 0.25f)));
    return r;
  }
  static __device__ __forceinline__ float fwd(float g, float u, const Consts&) {
    return ((g * 0.25f) * quarter_recip(g, g * g)) * u;
  }
  static __device__ __forceinline__ void bwd(float dh, float g, float u, const Consts&, float& dgate, float& dup) {
    const float x2 = g * g;
    const float sig = quarter_recip(g, x2) * 0.25f;
    dup = dh * (g * sig);
    const float dq = fmaf(x2, 3.0f * GeluConst::kQ3, GeluConst::kQ1);
    dgate = (dh * u) * (sig * fmaf(g * (1.0f - sig), dq, 1.0f));
  }
  // fwd and bwd of one element off one exponential; each result is the expression above, bit for bit
  static __device__ __forceinline__ void bwd_h(float dh, float g, float u, const Consts&, float& h, float& dgate,
                                               float& dup) {
    const float x2 = g * g;
    const float qr = quarter_recip(g, x2);
    const float sig = qr * 0.25f;
    h = ((g * 0.25f) * qr) * u;
    dup = dh * (g * sig);
    const float dq = fmaf(x2, 3.0f * GeluConst::kQ3, GeluConst::kQ1);
    dgate = (dh * u) * (sig * fmaf(g * (1.0f - sig), dq, 1.0f));
  }
};

template <> struct Math<false, ACT_GELU_TANH> {
  // 1 - s is formed as exp(-q) * s, which keeps its relative accuracy for large positive x (1 - s
  // itself would carry an absolute error that the derivative multiplies by x * q'(x), over a hundred
  // for |x| ~ 8); where exp(-q) overflows, s is 0 and 1 - s is 1.  The reciprocal of 1 + exp(-q) is
  // rcp.approx (at most 1 ulp off) as in Math<false, ACT_SILU>: two IEEE divisions per element held the
  // fp32 backward of [68298, 11008] at 6.64 TB/s.
  static __device__ __forceinline__ float fwd(float g, float u, const Consts&) {
    const float q = g * fmaf(g * g, GeluConst::kQ3, GeluConst::kQ1);
    return (g * Math<false, ACT_SILU>::recip(1.0f + expf(-q))) * u;
  }
  static __device__ __forceinline__ void bwd(float dh, float g, float u, const Consts&, float& dgate, float& dup) {
    const float x2 = g * g;
    const float q = g * fmaf(x2, GeluConst::kQ3, GeluConst::kQ1);
    const float e = expf(-q);
    const float sig = Math<false, ACT_SILU>::recip(1.0f + e);
    const float one_minus_sig = e < 1e30f ? e * sig : 1.0f;
    dup = dh * (g * sig);
    const float dq = fmaf(x2, 3.0f * GeluConst::kQ3, GeluConst::kQ1);
    dgate = (dh * u) * (sig * fmaf(g * one_minus_sig, dq, 1.0f));
  }
  static __device__ __forceinline__ void bwd_h(float dh, float g, float u, const Consts& c, float& h, float& dgate,
                                               float& dup) {
    h = fwd(g, u, c);  // same q, exp and reciprocal as bwd: the compiler shares them
    bwd(dh, g, u, c, dgate, dup);
  }
};

// 0.5 * P(t) of the erfc fit described at Math<true, ACT_GELU_ERF> (the halved coefficients are exact).
struct GeluErfcPoly {
  static __device__ __forceinline__ float half_p(float t) {
    float p = 0.5f * 0.0502124303f;
    p = fmaf(p, t, 0.5f * -0.182717498f);
    p = fmaf(p, t, 0.5f * 0.168813753f);
    p = fmaf(p, t, 0.5f * -0.00540429202f);
    p = fmaf(p, t, 0.5f * 0.14135102f);
    p = fmaf(p, t, 0.5f * 0.168557698f);
    p = fmaf(p, t, 0.5f * 0.207841563f);
    p = fmaf(p, t, 0.5f * 0.225669582f);
    p = fmaf(p, t, 0.5f * 0.225675864f);
    return p;
  }
};

// Exact form, fp32 I/O.  0.5 * erfc(|x| / sqrt 2) = 0.5 * t * P(t) * exp(-x^2 / 2) with the fit described at
// Math<true, ACT_GELU_ERF> below (relative error 2.5e-7 evaluated in fp32), but with the factors an fp32
// result needs: the exponent of exp(-x^2 / 2) carried in two parts (the rounding of x^2 alone would be a
// relative 1e-6 at |x| = 6) into one ex2.approx (2^-22), and a reciprocal that does not flush.  Every result
// stays within 1e-6 relative of the exact value.  erfcf and a second expf made this form compute-bound
// (forward 4.5 TB/s).
template <> struct Math<false, ACT_GELU_ERF> {
  static __device__ __forceinline__ void cdf_pdf(float x, float& cdf, float& pdf) {
    float t;
    asm("rcp.approx.f32 %0, %1;" : "=f"(t) : "f"(fmaf(fabsf(x), GeluConst::kErfcT, 1.0f)));
    // exp(-x^2 / 2) = 2^(th + tl): x^2 = hi + lo exactly, th the rounded product of hi and -log2(e) / 2, tl what
    // that rounding, the constant's own rounding and lo leave over (a few 1e-6 at most).  Where hi overflowed tl
    // is NaN and the minimum drops it (2^th is 0 there).
    const float hi = x * x;
    const float th = hi * -0.7213475108146667f;
    float tl = fmaf(hi, -0.7213475108146667f, -th);
    tl = fmaf(hi, -9.629815167500055e-09f, tl);
    tl = fmaf(fmaf(x, x, -hi), -0.7213475108146667f, tl);
    tl = fminf(tl, 1.0e-3f);
    float ex;
    asm("ex2.approx.f32 %0, %1;" : "=f"(ex) : "f"(th));
    ex = fmaf(ex, 0.6931471805599453f * tl, ex);
    const float half_erfc = t * GeluErfcPoly::half_p(t) * ex;  // 0.5 * erfc(|x| / sqrt 2)
    cdf = x < 0.0f ? half_erfc : 1.0f - half_erfc;
    pdf = GeluConst::kInvSqrt2Pi * ex;
  }
  static __device__ __forceinline__ float fwd(float g, float u, const Consts&) {
    float cdf, pdf;
    cdf_pdf(g, cdf, pdf);
    return (g * cdf) * u;
  }
  static __device__ __forceinline__ void bwd(float dh, float g, float u, const Consts&, float& dgate, float& dup) {
    float cdf, pdf;
    cdf_pdf(g, cdf, pdf);
    dup = dh * (g * cdf);
    dgate = (dh * u) * fmaf(g, pdf, cdf);
  }
  static __device__ __forceinline__ void bwd_h(float dh, float g, float u, const Consts&, float& h, float& dgate,
                                               float& dup) {
    float cdf, pdf;
    cdf_pdf(g, cdf, pdf);
    h = (g * cdf) * u;
    dup = dh * (g * cdf);
    dgate = (dh * u) * fmaf(g, pdf, cdf);
  }
};

// Exact form, 16-bit I/O.  erfcf costs ~40 instructions and made the kernel compute-bound (2.5 TB/s
// forward); here erfc(y) = t * P(t) * exp(-y^2) with t = 1 / (1 + 0.4 y) and P a degree-8 polynomial
// fitted to erfc(y) exp(y^2) / t in the relative sense over y in [0, inf): relative error < 3e-7
// everywhere, tail included, far below half an fp16 ulp.  The exp(-y^2) = exp(-x^2 / 2)
// factor is shared with the Gaussian density of the derivative.
template <> struct Math<true, ACT_GELU_ERF> {
  static __device__ __forceinline__ void cdf_pdf(float x, float& cdf, float& pdf) {
    float t, ex;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(fabsf(x), GeluConst::kErfcT, 1.0f)));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"((x * x) * (-0.5f * GeluConst::kLog2e)));
    const float half_erfc = t * GeluErfcPoly::half_p(t) * ex;  // 0.5 * erfc(|x| / sqrt 2)
    cdf = x < 0.0f ? half_erfc : 1.0f - half_erfc;
    pdf = GeluConst::kInvSqrt2Pi * ex;
  }
  static __device__ __forceinline__ float fwd(float g, float u, const Consts&) {
    float cdf, pdf;
    cdf_pdf(g, cdf, pdf);
    return (g * cdf) * u;
  }
  static __device__ __forceinline__ void bwd(float dh, float g, float u, const Consts&, float& dgate, float& dup) {
    float cdf, pdf;
    cdf_pdf(g, cdf, pdf);
    dup = dh * (g * cdf);
    dgate = (dh * u) * fmaf(g, pdf, cdf);
  }
  static __device__ __forceinline__ void bwd_h(float dh, float g, float u, const Consts&, float& h, float& dgate,
                                               float& dup) {
    float cdf, pdf;
    cdf_pdf(g, cdf, pdf);
    h = (g * cdf) * u;
    dup = dh * (g * cdf);
    dgate = (dh * u) * fmaf(g, pdf, cdf);
  }
};

// ---------------------------------------------------------------------------------------
// Work description shared by the forward and backward kernels.
//
// The body is `n_vec` vectors of BYTES bytes.  FLAT: vector i of every tensor sits at
// byte offset i*BYTES from that tensor's base.  ROWS: vector i belongs to row
// i / vecs_per_row, column-vector i % vecs_per_row; each tensor has its own row pitch in
// bytes (packed gate|up input of width 2I against an output of width I).
//
// FLAT launches also own up to `edge` scalar elements that did not fit the vector body:
// `head` elements in front of it (peeled so the body starts 16-byte aligned) and the rest
// behind it.
// ---------------------------------------------------------------------------------------

struct Shape {
  long long n_vec;         // vectors in the body
  long long vecs_per_row;  // ROWS only
  // ROWS only: i / vecs_per_row == __umulhi(i, div_mul) >> div_shift for every i < 2^31 (div_mul == 0: not
  // available, divide); see set_row_divisor().
  unsigned div_mul, div_shift;
  long long pitch_in;      // bytes between rows of gate / up                (ROWS only)
  long long pitch_out;     // bytes between rows of h (fwd) or dh (bwd)      (ROWS only)
  long long pitch_grad;    // bytes between rows of dgate / dup              (ROWS, bwd only)
  int head;                // scalar elements before the body                (FLAT only)
  int edge;                // head + tail scalar elements                    (FLAT only)
  // SHIFT kernels only: how many bytes past a 16-byte boundary the body of each INPUT starts, when
  // the outputs' bodies start on one (0..15, a multiple of the element size).
  int skew_gate, skew_up, skew_dout;
};

// Division of a vector index by vecs_per_row as a multiplication: with p = 31 + ceil(log2 d) and
// m = ceil(2^p / d) (which fits 32 bits), floor(i / d) = (i * m) >> p for every 0 <= i < 2^31 (Granlund and
// Montgomery's invariant-divisor scheme).  Left at zero, i.e. "divide", where that range does not cover the launch.
inline void set_row_divisor(Shape& s) {
  s.div_mul = s.div_shift = 0;
  const unsigned long long d = (unsigned long long)s.vecs_per_row;
  if (d < 2 || d >= (1ull << 31) || s.n_vec >= (1ll << 31)) return;
  unsigned lg = 0;
  while ((1ull << lg) < d) ++lg;
  const unsigned p = 31 + lg;
  s.div_mul = (unsigned)(((1ull << p) + d - 1) / d);
  s.div_shift = p - 32;
}

// ---------------------------------------------------------------------------------------
// Loads for inputs that are misaligned relative to the outputs (flat layout, 16-byte vectors; used by the
// backward -- the forward reads skewed inputs through the ragged-row kernel further down).
// Vector i of such an input straddles two aligned 16-byte granules.  Every thread loads the granule its
// vector mostly lies in with one aligned access, plus the one or two 32-bit words of the neighbouring granule
// that complete it: the adjacent lane loads that granule as its own, so the second access hits L1 (skewed
// inputs are therefore read with plain, L1-allocating loads).  The words are then funnel-shifted into place.
// Bytes outside the tensor that share a granule with its first or last element are read and discarded.
// (Passing the neighbouring words between lanes by shuffle instead, with the warp's edge lanes fetching their
// own, was 4-10 % slower: width 11009, dh/gate/up 2 / 8 / 14 bytes off: 6.71 / 6.26 / 6.09 TB/s against
// 6.99 / 6.71 / 6.70 now.)
// ---------------------------------------------------------------------------------------

static __device__ __forceinline__ const char* cbyte(const void* p) { return static_cast<const char*>(p); }
static __device__ __forceinline__ char* byte(void* p) { return static_cast<char*>(p); }

__device__ __forceinline__ Vec<16> funnel16(const Vec<16>& lo, const Vec<16>& hi, int skew) {
  const uint32_t w[8] = {lo.w[0], lo.w[1], lo.w[2], lo.w[3], hi.w[0], hi.w[1], hi.w[2], hi.w[3]};
  const int sh = (skew & 3) * 8;
  Vec<16> o;
  switch (skew >> 2) {  // uniform over the launch
    case 0:
#pragma unroll
      for (int i = 0; i < 4; ++i) o.w[i] = __funnelshift_r(w[i], w[i + 1], sh);
      break;
    case 1:
#pragma unroll
      for (int i = 0; i < 4; ++i) o.w[i] = __funnelshift_r(w[i + 1], w[i + 2], sh);
      break;
    case 2:
#pragma unroll
      for (int i = 0; i < 4; ++i) o.w[i] = __funnelshift_r(w[i + 2], w[i + 3], sh);
      break;
    default:
#pragma unroll
      for (int i = 0; i < 4; ++i) o.w[i] = __funnelshift_r(w[i + 3], w[i + 4], sh);
      break;
  }
  return o;
}

// NW = how many 32-bit words of the NEIGHBOURING granule a vector takes besides its main granule.  The main
// granule is the one the vector starts in when the skew is at most 8 bytes (the words are the first of the NEXT
// granule) and the one it ends in otherwise (the last words of the PREVIOUS granule), so two words always suffice
// (NW = 2).  NW = 1 serves launches whose inputs are all within 4 bytes of a boundary in either direction (one
// element off, the common case) and leaves registers for one more tile row in flight.
//
// Phase 1, with the other loads of the tile: `base` is the input's body pointer (misaligned by `skew` bytes), `off`
// the byte offset of vector i in the outputs.  LDM is the load mode of an input that is not skewed.
template <int LDM, int NW>
__device__ __forceinline__ void ld_skewed_issue(const void* base, long long off, int skew, bool active, Vec<16>& lo,
                                                Vec<4 * NW>& nb) {
  lo = Vec<16>{};
  nb = Vec<4 * NW>{};
  if (!active) return;
  const char* granule = cbyte(base) - skew + off;  // the aligned granule the vector starts in
  if (skew == 0) {  // uniform over the launch, like the branches below
    lo = Ld<16, LDM>::ld(granule);
  } else if (skew > 8) {
    nb = Ld<4 * NW, LD_PLAIN>::ld(granule + 16 - 4 * NW);
    lo = Ld<16, LD_PLAIN>::ld(granule + 16);
  } else {
    lo = Ld<16, LD_PLAIN>::ld(granule);
    nb = Ld<4 * NW, LD_PLAIN>::ld(granule + 16);
  }
}

// Phase 2, after every load of the tile has been issued.
template <int NW>
__device__ __forceinline__ Vec<16> ld_skewed_finish(const Vec<16>& lo, const Vec<4 * NW>& nb, int skew) {
  if (skew == 0) return lo;
  Vec<16> other{};
  if (skew > 8) {
#pragma unroll
    for (int i = 0; i < NW; ++i) other.w[4 - NW + i] = nb.w[i];
    return funnel16(other, lo, skew);
  }
#pragma unroll
  for (int i = 0; i < NW; ++i) other.w[i] = nb.w[i];
  return funnel16(lo, other, skew);
}

template <bool ROWS, int BYTES>
struct Locator {
  // Byte offsets of vector `i` in the three pitch classes.
  static __device__ __forceinline__ void at(const Shape& s, long long i, long long& off_in, long long& off_out,
                                            long long& off_grad) {
    if constexpr (!ROWS) {
      off_in = off_out = off_grad = i * BYTES;
    } else {
      long long row, cv;
      if (s.div_mul != 0) {  // uniform branch; a multiplication and a shift instead of a division
        const unsigned r = __umulhi((unsigned)i, s.div_mul) >> s.div_shift;
        row = r;
        cv = (long long)((unsigned)i - r * (unsigned)s.vecs_per_row);
      } else if (s.n_vec <= 0xffffffffLL) {  // 32-bit division is several times cheaper than 64-bit
        unsigned r = (unsigned)i / (unsigned)s.vecs_per_row;
        row = r;
        cv = (long long)((unsigned)i - r * (unsigned)s.vecs_per_row);
      } else {
        row = i / s.vecs_per_row;
        cv = i - row * s.vecs_per_row;
      }
      off_in = row * s.pitch_in + cv * BYTES;
      off_out = row * s.pitch_out + cv * BYTES;
      off_grad = row * s.pitch_grad + cv * BYTES;
    }
  }
};

// ---------------------------------------------------------------------------------------
// Forward.  One tile = THREADS*UNROLL vectors; thread t owns vectors t, t+THREADS, ... of
// the tile, so each warp-wide access is one contiguous 512- or 1024-byte segment.
// ---------------------------------------------------------------------------------------

template <class T, int BYTES, bool FAST, bool ROWS, int THREADS, int UNROLL, int LDM, int STM, int ACT = ACT_SILU>
__global__ void __launch_bounds__(THREADS, 2)  // two 512-thread CTAs per SM: at most 64 registers
swiglu_fwd_kernel(void* __restrict__ out, const void* __restrict__ gate, const void* __restrict__ up, Shape s,
                  float gm, float dm) {
  constexpr int EPV = BYTES / Codec<T>::kSize;
  constexpr long long TILE = (long long)THREADS * UNROLL;
  const long long n_tiles = (s.n_vec + TILE - 1) / TILE;
  const Consts c(gm, dm);

  for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const long long v0 = tile * TILE + threadIdx.x;
    const bool full = (tile + 1) * TILE <= s.n_vec;
    Vec<BYTES> g[UNROLL], u[UNROLL];
    long long oo[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const long long i = v0 + (long long)k * THREADS;
      if (full || i < s.n_vec) {
        long long oi, og;
        Locator<ROWS, BYTES>::at(s, i, oi, oo[k], og);
        g[k] = Ld<BYTES, LDM>::ld(cbyte(gate) + oi);
        u[k] = Ld<BYTES, LDM>::ld(cbyte(up) + oi);
      }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const long long i = v0 + (long long)k * THREADS;
      if (full || i < s.n_vec) {
        float fg[EPV], fu[EPV], fh[EPV];
        Codec<T>::template unpack<BYTES>(g[k], fg);
        Codec<T>::template unpack<BYTES>(u[k], fu);
#pragma unroll
        for (int e = 0; e < EPV; ++e) fh[e] = Math<FAST, ACT>::fwd(fg[e], fu[e], c);
        Vec<BYTES> h;
        Codec<T>::template pack<BYTES>(fh, h);
        St<BYTES, STM>::st(byte(out) + oo[k], h);
      }
    }
  }

  if constexpr (!ROWS) {
    // Ragged edges of a flat stream: at most 2*(16/sizeof(T) - 1) scalar elements.
    if (blockIdx.x == gridDim.x - 1 && (int)threadIdx.x < s.edge) {
      constexpr int ES = Codec<T>::kSize;
      const int t = threadIdx.x;
      const long long idx = t < s.head ? (long long)t : (long long)t + s.n_vec * EPV;
      // Element idx of the launch's logical stream; the body pointers were advanced past
      // the head by the host, so address relative to them is (idx - head).
      const long long off = (idx - s.head) * ES;
      Vec<ES> vg = Ld<ES, LD_PLAIN>::ld(cbyte(gate) + off);
      Vec<ES> vu = Ld<ES, LD_PLAIN>::ld(cbyte(up) + off);
      float fg[1], fu[1], fh[1];
      Codec<T>::template unpack<ES>(vg, fg);
      Codec<T>::template unpack<ES>(vu, fu);
      fh[0] = Math<FAST, ACT>::fwd(fg[0], fu[0], c);
      Vec<ES> vh;
      Codec<T>::template pack<ES>(fh, vh);
      St<ES, ST_PLAIN>::st(byte(out) + off, vh);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Backward.  LDM_IO is the load mode of gate/up: it must be a coherent mode whenever
// dgate/dup alias them.  dh is always read-only.
// ---------------------------------------------------------------------------------------

template <class T, int BYTES, bool FAST, bool ROWS, int THREADS, int UNROLL, int LDM_DH, int LDM_IO, int STM,
          int SHIFT = 0, int ACT = ACT_SILU>
__global__ void __launch_bounds__(THREADS, 2)
swiglu_bwd_kernel(void* dgate, void* dup, const void* __restrict__ dout, const void* gate, const void* up, Shape s,
                  float gm, float dm) {
  constexpr int EPV = BYTES / Codec<T>::kSize;
  constexpr long long TILE = (long long)THREADS * UNROLL;
  const long long n_tiles = (s.n_vec + TILE - 1) / TILE;
  const Consts c(gm, dm);

  for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const long long v0 = tile * TILE + threadIdx.x;
    const bool full = (tile + 1) * TILE <= s.n_vec;
    Vec<BYTES> d[UNROLL], g[UNROLL], u[UNROLL];
    constexpr int NW = SHIFT ? SHIFT : 1;
    Vec<4 * NW> d2[SHIFT ? UNROLL : 1], g2[SHIFT ? UNROLL : 1], u2[SHIFT ? UNROLL : 1];
    long long og[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const long long i = v0 + (long long)k * THREADS;
      if constexpr (SHIFT) {
        static_assert(!SHIFT || (BYTES == 16 && !ROWS), "skewed loads exist for flat 16-byte streams only");
        const bool active = full || i < s.n_vec;
        og[k] = i * BYTES;
        ld_skewed_issue<LDM_DH, NW>(dout, og[k], s.skew_dout, active, d[k], d2[k]);
        ld_skewed_issue<LDM_IO, NW>(gate, og[k], s.skew_gate, active, g[k], g2[k]);
        ld_skewed_issue<LDM_IO, NW>(up, og[k], s.skew_up, active, u[k], u2[k]);
      } else if (full || i < s.n_vec) {
        long long oi, oo;
        Locator<ROWS, BYTES>::at(s, i, oi, oo, og[k]);
        d[k] = Ld<BYTES, LDM_DH>::ld(cbyte(dout) + oo);
        g[k] = Ld<BYTES, LDM_IO>::ld(cbyte(gate) + oi);
        u[k] = Ld<BYTES, LDM_IO>::ld(cbyte(up) + oi);
      }
    }
    // All loads of the tile are issued (volatile asm keeps program order) before the first
    // store below, so an in-place launch never reads a vector it has already overwritten.
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const long long i = v0 + (long long)k * THREADS;
      if constexpr (SHIFT) {
        d[k] = ld_skewed_finish<NW>(d[k], d2[k], s.skew_dout);
        g[k] = ld_skewed_finish<NW>(g[k], g2[k], s.skew_gate);
        u[k] = ld_skewed_finish<NW>(u[k], u2[k], s.skew_up);
      }
      if (full || i < s.n_vec) {
        float fd[EPV], fg[EPV], fu[EPV], fdg[EPV], fdu[EPV];
        Codec<T>::template unpack<BYTES>(d[k], fd);
        Codec<T>::template unpack<BYTES>(g[k], fg);
        Codec<T>::template unpack<BYTES>(u[k], fu);
#pragma unroll
        for (int e = 0; e < EPV; ++e) Math<FAST, ACT>::bwd(fd[e], fg[e], fu[e], c, fdg[e], fdu[e]);
        Vec<BYTES> vdg, vdu;
        Codec<T>::template pack<BYTES>(fdg, vdg);
        Codec<T>::template pack<BYTES>(fdu, vdu);
        St<BYTES, STM>::st(byte(dgate) + og[k], vdg);
        St<BYTES, STM>::st(byte(dup) + og[k], vdu);
      }
    }
  }

  if constexpr (!ROWS) {
    if (blockIdx.x == gridDim.x - 1 && (int)threadIdx.x < s.edge) {
      constexpr int ES = Codec<T>::kSize;
      const int t = threadIdx.x;
      const long long idx = t < s.head ? (long long)t : (long long)t + s.n_vec * EPV;
      const long long off = (idx - s.head) * ES;
      Vec<ES> vd = Ld<ES, LD_PLAIN>::ld(cbyte(dout) + off);
      Vec<ES> vg = Ld<ES, LD_PLAIN>::ld(cbyte(gate) + off);
      Vec<ES> vu = Ld<ES, LD_PLAIN>::ld(cbyte(up) + off);
      float fd[1], fg[1], fu[1], fdg[1], fdu[1];
      Codec<T>::template unpack<ES>(vd, fd);
      Codec<T>::template unpack<ES>(vg, fg);
      Codec<T>::template unpack<ES>(vu, fu);
      Math<FAST, ACT>::bwd(fd[0], fg[0], fu[0], c, fdg[0], fdu[0]);
      Vec<ES> vdg, vdu;
      Codec<T>::template pack<ES>(fdg, vdg);
      Codec<T>::template pack<ES>(fdu, vdu);
      St<ES, ST_PLAIN>::st(byte(dgate) + off, vdg);
      St<ES, ST_PLAIN>::st(byte(dup) + off, vdu);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Ragged rows: wide accesses for layouts in which no two tensors, and no two rows of one tensor,
// need share an alignment -- pitched rows whose pitch or width is not a multiple of 16 bytes (the
// packed gate|up layout with an odd half-width: the up half of every row is skewed against the
// gate half, and every row against the previous one) and flat tensors whose two outputs are skewed
// against each other.
//
// The unit is a 32-byte FRAME (32-byte aligned).  A row is cut by its PRIMARY output (h forward,
// dgate backward): `head` scalar elements up to the first frame boundary, `nv` whole frames,
// `tail` scalar elements.  One warp TASK is 32 consecutive frames of one row, one per lane, so
// everything about the row's alignment is uniform over the warp and worked out once per task; a
// CTA is a few consecutive tasks of one row, and the grid's y/z give the row (no division).
// The last task of a row also takes the head and tail elements, one per lane.
//
// An input whose row body starts `s` bytes past a frame boundary is read as the frame the vector
// mostly lies in (one 32-byte load) plus the adjoining 16 bytes of the neighbouring frame (the
// next lane loads that frame anyway, so the line is in flight or in L1), and the 48-byte window is
// funnel-shifted into place: no shuffles, no edge lanes.  The SECONDARY output of the backward
// (dup) goes the other way: a lane builds the aligned frame its vector starts (s <= 16) or ends
// (s > 16) in from its own words and four words of the neighbouring lane, and the first and last
// lane of a task store the bytes that are left over in aligned pieces of 16, 8, 4 and 2 bytes.  No
// byte is written that is not the launch's own, so guard bands survive.
//
// In place (dgate == gate, dup == up): every lane issues all its loads before its first store,
// the warp converges (the shuffles of the dup store) between the two, and the bytes a lane reads
// from a frame that a lane of ANOTHER warp may already have written are bytes it discards.
// ---------------------------------------------------------------------------------------

struct RaggedShape {
  long long rows, cols;  // elements
  int tasks_per_row;     // warp tasks (32 frames each) per row
  long long pitch_in;    // bytes between rows of gate / up
  long long pitch_out;   // bytes between rows of h (fwd) or dh (bwd)
  long long pitch_grad;  // bytes between rows of dgate / dup (bwd only)
};

// How a row is cut, from the address of its primary output.
struct RaggedRow {
  int head, tail;  // scalar elements before / after the body
  long long nv;    // frames in the body
};

template <int ES>
__device__ __forceinline__ RaggedRow ragged_row(long long cols, const void* primary_row) {
  constexpr int EPV = 32 / ES;
  RaggedRow r;
  long long head = (long long)((32u - (unsigned)((uintptr_t)primary_row & 31u)) & 31u) / ES;
  if (head > cols) head = cols;
  r.head = (int)head;
  r.nv = (cols - head) / EPV;
  r.tail = (int)(cols - head - r.nv * EPV);
  return r;
}

// Bytes [q, q + 32) of the 48-byte window w[0..11], q a multiple of 2 in [0, 16] (uniform over the warp).
__device__ __forceinline__ Vec<32> shift_window(const uint32_t (&w)[12], int q) {
  const int sh = (q & 3) * 8;
  Vec<32> o;
  switch (q >> 2) {
    case 0:
#pragma unroll
      for (int i = 0; i < 8; ++i) o.w[i] = __funnelshift_r(w[i], w[i + 1], sh);
      break;
    case 1:
#pragma unroll
      for (int i = 0; i < 8; ++i) o.w[i] = __funnelshift_r(w[i + 1], w[i + 2], sh);
      break;
    case 2:
#pragma unroll
      for (int i = 0; i < 8; ++i) o.w[i] = __funnelshift_r(w[i + 2], w[i + 3], sh);
      break;
    case 3:
#pragma unroll
      for (int i = 0; i < 8; ++i) o.w[i] = __funnelshift_r(w[i + 3], w[i + 4], sh);
      break;
    default:  // q == 16
#pragma unroll
      for (int i = 0; i < 8; ++i) o.w[i] = w[i + 4];
      break;
  }
  return o;
}

// A vector read through a window: `main` is the frame it mostly lies in, `nb` the adjoining half of the other.
struct Window {
  Vec<32> main;
  Vec<16> nb;
};

// `body` is the row's body in this tensor (s = body & 31 bytes past a frame boundary), `v` the frame index.
template <int LDM>
__device__ __forceinline__ void ld_window_issue(const char* body, long long v, int s, bool active, Window& w) {
  if (!active) return;
  const char* frame = body - s + v * 32;  // the aligned frame the vector starts in
  if (s == 0) {
    w.main = Ld<32, LDM>::ld(frame);
  } else if (s <= 16) {
    w.main = Ld<32, LDM>::ld(frame);
    w.nb = Ld<16, LDM>::ld(frame + 32);  // first half of the next frame
  } else {
    w.nb = Ld<16, LDM>::ld(frame + 16);  // second half of this frame
    w.main = Ld<32, LDM>::ld(frame + 32);
  }
}

__device__ __forceinline__ Vec<32> ld_window_finish(const Window& w, int s) {
  if (s == 0) return w.main;  // uniform over the warp, like the two branches below
  if (s <= 16) {
    const uint32_t x[12] = {w.main.w[0], w.main.w[1], w.main.w[2], w.main.w[3], w.main.w[4], w.main.w[5],
                            w.main.w[6], w.main.w[7], w.nb.w[0],   w.nb.w[1],   w.nb.w[2],   w.nb.w[3]};
    return shift_window(x, s);
  }
  const uint32_t x[12] = {w.nb.w[0],   w.nb.w[1],   w.nb.w[2],   w.nb.w[3],   w.main.w[0], w.main.w[1],
                          w.main.w[2], w.main.w[3], w.main.w[4], w.main.w[5], w.main.w[6], w.main.w[7]};
  return shift_window(x, s - 16);
}

// Stores bytes [A, B) of the aligned frame image `f` to frame + A .. frame + B in the fewest aligned pieces
// (16, 8, 4, 2 bytes); A and B are compile-time, so every register index is static.
template <int A, int B>
__device__ __forceinline__ void st_frame_static(char* frame, const Vec<32>& f) {
  if constexpr (A < B) {
    constexpr int room = B - A;
    constexpr int size = ((A & 15) == 0 && room >= 16) ? 16 : ((A & 7) == 0 && room >= 8) ? 8
                         : ((A & 3) == 0 && room >= 4) ? 4 : 2;
    if constexpr (size == 16) {
      Vec<16> x;
      x.w[0] = f.w[A / 4], x.w[1] = f.w[A / 4 + 1], x.w[2] = f.w[A / 4 + 2], x.w[3] = f.w[A / 4 + 3];
      St<16, ST_PLAIN>::st(frame + A, x);
    } else if constexpr (size == 8) {
      Vec<8> x;
      x.w[0] = f.w[A / 4], x.w[1] = f.w[A / 4 + 1];
      St<8, ST_PLAIN>::st(frame + A, x);
    } else if constexpr (size == 4) {
      Vec<4> x;
      x.w[0] = f.w[A / 4];
      St<4, ST_PLAIN>::st(frame + A, x);
    } else {
      Vec<2> x;
      x.w[0] = (A & 2) ? (f.w[A / 4] >> 16) : (f.w[A / 4] & 0xffffu);
      St<2, ST_PLAIN>::st(frame + A, x);
    }
    st_frame_static<A + size, B>(frame, f);
  }
}

// Bytes [s, 32) of the frame image (TAIL) or bytes [0, s) (not TAIL); s a multiple of 2 in (0, 32), uniform over
// the warp: one jump, then at most four stores with static registers.  Edge lanes of a task only.
template <bool TAIL>
__device__ __forceinline__ void st_frame_part(char* frame, const Vec<32>& f, int s) {
#define SWIGLU_FRAME_CASE(S)                                   \
  case S:                                                      \
    if constexpr (TAIL) st_frame_static<S, 32>(frame, f);      \
    else st_frame_static<0, S>(frame, f);                      \
    break;
  switch (s) {
    SWIGLU_FRAME_CASE(2) SWIGLU_FRAME_CASE(4) SWIGLU_FRAME_CASE(6) SWIGLU_FRAME_CASE(8) SWIGLU_FRAME_CASE(10)
    SWIGLU_FRAME_CASE(12) SWIGLU_FRAME_CASE(14) SWIGLU_FRAME_CASE(16) SWIGLU_FRAME_CASE(18) SWIGLU_FRAME_CASE(20)
    SWIGLU_FRAME_CASE(22) SWIGLU_FRAME_CASE(24) SWIGLU_FRAME_CASE(26) SWIGLU_FRAME_CASE(28) SWIGLU_FRAME_CASE(30)
    default: break;
  }
#undef SWIGLU_FRAME_CASE
}

// Lane l holds vector `v` whose destination `dst` lies `s` bytes past a frame boundary.  All 32 lanes must call
// this together.  `first`: the lane has no preceding lane with a vector of the same run (lane 0); `last`: none
// following (lane 31 or the row's last frame).
template <int STM>
__device__ __forceinline__ void st_skewed32(char* dst, const Vec<32>& v, int s, bool active, bool first, bool last) {
  if (s == 0) {  // uniform over the warp
    if (active) St<32, STM>::st(dst, v);
    return;
  }
  char* frame = dst - s;  // the aligned frame the vector starts in; it ends in the next one
  if (s <= 16) {
    // the frame it starts in = the last s bytes of the previous lane's vector, then the first 32 - s of ours
    uint32_t p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __shfl_up_sync(0xffffffffu, v.w[4 + i], 1);
    if (!active) return;
    const uint32_t x[12] = {p[0], p[1], p[2], p[3], v.w[0], v.w[1], v.w[2], v.w[3], v.w[4], v.w[5], v.w[6], v.w[7]};
    const Vec<32> start = shift_window(x, 16 - s);
    if (!first) St<32, STM>::st(frame, start);
    else st_frame_part<true>(frame, start, s);
    if (last) {  // our last s bytes open the next frame
      const uint32_t y[12] = {v.w[4], v.w[5], v.w[6], v.w[7], 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      st_frame_part<false>(frame + 32, shift_window(y, 16 - s), s);
    }
  } else {
    // the frame it ends in = our last s bytes, then the first 32 - s bytes of the next lane's vector
    uint32_t n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = __shfl_down_sync(0xffffffffu, v.w[i], 1);
    if (!active) return;
    const uint32_t x[12] = {v.w[0], v.w[1], v.w[2], v.w[3], v.w[4], v.w[5], v.w[6], v.w[7], n[0], n[1], n[2], n[3]};
    const Vec<32> end = shift_window(x, 32 - s);
    if (!last) St<32, STM>::st(frame + 32, end);
    else st_frame_part<false>(frame + 32, end, s);
    if (first) {  // our first 32 - s bytes close the frame before
      const uint32_t y[12] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, v.w[0], v.w[1], v.w[2], v.w[3]};
      st_frame_part<true>(frame, shift_window(y, 32 - s), s);
    }
  }
}

// Row of this CTA (grid y/z) and frame of this lane (grid x, warp, lane).
struct RaggedCoord {
  long long row;
  long long v;
  bool last_task;
};
__device__ __forceinline__ RaggedCoord ragged_coord(const RaggedShape& s) {
  RaggedCoord c;
  c.row = (long long)blockIdx.y + (long long)blockIdx.z * gridDim.y;
  const int task = (int)blockIdx.x * (int)(blockDim.x >> 5) + (int)(threadIdx.x >> 5);
  c.v = (long long)task * 32 + (threadIdx.x & 31);
  c.last_task = task == s.tasks_per_row - 1;
  return c;
}

template <class T, bool FAST, int MAX_THREADS, int MIN_CTAS, int LDM, int STM, int ACT = ACT_SILU>
__global__ void __launch_bounds__(MAX_THREADS, MIN_CTAS)
swiglu_fwd_ragged_kernel(void* out, const void* __restrict__ gate, const void* __restrict__ up, RaggedShape s,
                         float gm, float dm) {
  constexpr int ES = Codec<T>::kSize;
  constexpr int EPV = 32 / ES;
  const RaggedCoord at = ragged_coord(s);
  if (at.row >= s.rows) return;
  const Consts c(gm, dm);
  const char* out_row = cbyte(out) + at.row * s.pitch_out;
  const RaggedRow r = ragged_row<ES>(s.cols, out_row);
  const long long hb = (long long)r.head * ES;
  const char* pg = cbyte(gate) + at.row * s.pitch_in + hb;  // the row's body in each tensor
  const char* pu = cbyte(up) + at.row * s.pitch_in + hb;
  char* po = byte(out) + at.row * s.pitch_out + hb;
  const int skew_g = (int)((uintptr_t)pg & 31), skew_u = (int)((uintptr_t)pu & 31);
  const bool active = at.v < r.nv;
  Window g, u;
  ld_window_issue<LDM>(pg, at.v, skew_g, active, g);
  ld_window_issue<LDM>(pu, at.v, skew_u, active, u);
  const int lane = threadIdx.x & 31;
  const bool scalar = at.last_task && lane < r.head + r.tail;
  // element of the row this lane takes as a scalar, relative to the body (negative: head)
  const long long eo = ((lane < r.head ? (long long)lane : (long long)lane + r.nv * EPV) - r.head) * ES;
  Vec<ES> sg{}, su{};
  if (scalar) {
    sg = Ld<ES, LD_PLAIN>::ld(pg + eo);
    su = Ld<ES, LD_PLAIN>::ld(pu + eo);
  }
  if (active) {
    const Vec<32> vg = ld_window_finish(g, skew_g), vu = ld_window_finish(u, skew_u);
    float fg[EPV], fu[EPV], fh[EPV];
    Codec<T>::template unpack<32>(vg, fg);
    Codec<T>::template unpack<32>(vu, fu);
#pragma unroll
    for (int e = 0; e < EPV; ++e) fh[e] = Math<FAST, ACT>::fwd(fg[e], fu[e], c);
    Vec<32> h;
    Codec<T>::template pack<32>(fh, h);
    St<32, STM>::st(po + at.v * 32, h);
  }
  if (scalar) {
    float fg[1], fu[1], fh[1];
    Codec<T>::template unpack<ES>(sg, fg);
    Codec<T>::template unpack<ES>(su, fu);
    fh[0] = Math<FAST, ACT>::fwd(fg[0], fu[0], c);
    Vec<ES> vh;
    Codec<T>::template pack<ES>(fh, vh);
    St<ES, ST_PLAIN>::st(po + eo, vh);
  }
}

template <class T, bool FAST, int MAX_THREADS, int MIN_CTAS, int LDM_DH, int LDM_IO, int STM, int ACT = ACT_SILU>
__global__ void __launch_bounds__(MAX_THREADS, MIN_CTAS)
swiglu_bwd_ragged_kernel(void* dgate, void* dup, const void* __restrict__ dout, const void* gate, const void* up,
                         RaggedShape s, float gm, float dm) {
  constexpr int ES = Codec<T>::kSize;
  constexpr int EPV = 32 / ES;
  const RaggedCoord at = ragged_coord(s);
  if (at.row >= s.rows) return;  // whole CTA
  const Consts c(gm, dm);
  const RaggedRow r = ragged_row<ES>(s.cols, cbyte(dgate) + at.row * s.pitch_grad);
  const long long hb = (long long)r.head * ES;
  const char* pd = cbyte(dout) + at.row * s.pitch_out + hb;  // the row's body in each tensor
  const char* pg = cbyte(gate) + at.row * s.pitch_in + hb;
  const char* pu = cbyte(up) + at.row * s.pitch_in + hb;
  char* pdg = byte(dgate) + at.row * s.pitch_grad + hb;
  char* pdu = byte(dup) + at.row * s.pitch_grad + hb;
  const int skew_d = (int)((uintptr_t)pd & 31), skew_g = (int)((uintptr_t)pg & 31);
  const int skew_u = (int)((uintptr_t)pu & 31), skew_du = (int)((uintptr_t)pdu & 31);
  const int lane = threadIdx.x & 31;
  const bool active = at.v < r.nv;
  const bool last = lane == 31 || at.v + 1 >= r.nv;
  Window d, g, u;
  ld_window_issue<LDM_DH>(pd, at.v, skew_d, active, d);
  ld_window_issue<LDM_IO>(pg, at.v, skew_g, active, g);
  ld_window_issue<LDM_IO>(pu, at.v, skew_u, active, u);
  const bool scalar = at.last_task && lane < r.head + r.tail;
  const long long eo = ((lane < r.head ? (long long)lane : (long long)lane + r.nv * EPV) - r.head) * ES;
  Vec<ES> sd{}, sg{}, su{};
  if (scalar) {  // loaded with everything else, before any store of this lane
    sd = Ld<ES, LD_PLAIN>::ld(pd + eo);
    sg = Ld<ES, LD_PLAIN>::ld(pg + eo);
    su = Ld<ES, LD_PLAIN>::ld(pu + eo);
  }
  Vec<32> vdu{};
  if (active) {
    const Vec<32> vd = ld_window_finish(d, skew_d), vg = ld_window_finish(g, skew_g), vu = ld_window_finish(u, skew_u);
    float fd[EPV], fg[EPV], fu[EPV], fdg[EPV], fdu[EPV];
    Codec<T>::template unpack<32>(vd, fd);
    Codec<T>::template unpack<32>(vg, fg);
    Codec<T>::template unpack<32>(vu, fu);
#pragma unroll
    for (int e = 0; e < EPV; ++e) Math<FAST, ACT>::bwd(fd[e], fg[e], fu[e], c, fdg[e], fdu[e]);
    Vec<32> vdg;
    Codec<T>::template pack<32>(fdg, vdg);
    Codec<T>::template pack<32>(fdu, vdu);
    St<32, STM>::st(pdg + at.v * 32, vdg);
  }
  st_skewed32<STM>(pdu + at.v * 32, vdu, skew_du, active, lane == 0, last);
  if (scalar) {
    float fd[1], fg[1], fu[1], fdg[1], fdu[1];
    Codec<T>::template unpack<ES>(sd, fd);
    Codec<T>::template unpack<ES>(sg, fg);
    Codec<T>::template unpack<ES>(su, fu);
    Math<FAST, ACT>::bwd(fd[0], fg[0], fu[0], c, fdg[0], fdu[0]);
    Vec<ES> xdg, xdu;
    Codec<T>::template pack<ES>(fdg, xdg);
    Codec<T>::template pack<ES>(fdu, xdu);
    St<ES, ST_PLAIN>::st(pdg + eo, xdg);
    St<ES, ST_PLAIN>::st(pdu + eo, xdu);
  }
}

// ---------------------------------------------------------------------------------------
// Backward that also recomputes the forward output: (h, dgate, dup) from (dh, gate, up) in one
// pass over flat, equally laid out tensors -- what a training step that kept gate and up but
// not h needs (the LoRA-MLP backward, whose down-projection adapter gradients contract with h).
// Every thread loads its three vectors before it stores, so each output may overwrite any one
// of the inputs exactly; LDM must then be a coherent load mode.  `n_vec` vectors of BYTES
// bytes, then `tail` scalar elements handled by the last CTA.
// ---------------------------------------------------------------------------------------

template <class T, int BYTES, bool FAST, int THREADS, int UNROLL, int LDM, int STM, int ACT = ACT_SILU>
__global__ void __launch_bounds__(THREADS)
swiglu_bwd_recompute_kernel(void* h, void* dgate, void* dup, const void* dout, const void* gate, const void* up,
                            long long n_vec, int tail, float gm, float dm) {
  constexpr int EPV = BYTES / Codec<T>::kSize;
  constexpr long long TILE = (long long)THREADS * UNROLL;
  const long long n_tiles = (n_vec + TILE - 1) / TILE;
  const Consts c(gm, dm);

  for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const long long v0 = tile * TILE + threadIdx.x;
    const bool full = (tile + 1) * TILE <= n_vec;
    Vec<BYTES> d[UNROLL], g[UNROLL], u[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const long long i = v0 + (long long)k * THREADS;
      if (full || i < n_vec) {
        d[k] = Ld<BYTES, LDM>::ld(cbyte(dout) + i * BYTES);
        g[k] = Ld<BYTES, LDM>::ld(cbyte(gate) + i * BYTES);
        u[k] = Ld<BYTES, LDM>::ld(cbyte(up) + i * BYTES);
      }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const long long i = v0 + (long long)k * THREADS;
      if (full || i < n_vec) {
        float fd[EPV], fg[EPV], fu[EPV], fh[EPV], fdg[EPV], fdu[EPV];
        Codec<T>::template unpack<BYTES>(d[k], fd);
        Codec<T>::template unpack<BYTES>(g[k], fg);
        Codec<T>::template unpack<BYTES>(u[k], fu);
#pragma unroll
        for (int e = 0; e < EPV; ++e) Math<FAST, ACT>::bwd_h(fd[e], fg[e], fu[e], c, fh[e], fdg[e], fdu[e]);
        Vec<BYTES> vh, vdg, vdu;
        Codec<T>::template pack<BYTES>(fh, vh);
        Codec<T>::template pack<BYTES>(fdg, vdg);
        Codec<T>::template pack<BYTES>(fdu, vdu);
        St<BYTES, STM>::st(byte(h) + i * BYTES, vh);
        St<BYTES, STM>::st(byte(dgate) + i * BYTES, vdg);
        St<BYTES, STM>::st(byte(dup) + i * BYTES, vdu);
      }
    }
  }

  if (blockIdx.x == gridDim.x - 1 && (int)threadIdx.x < tail) {
    constexpr int ES = Codec<T>::kSize;
    const long long off = (n_vec * EPV + threadIdx.x) * ES;
    Vec<ES> vd = Ld<ES, LD_PLAIN>::ld(cbyte(dout) + off);
    Vec<ES> vg = Ld<ES, LD_PLAIN>::ld(cbyte(gate) + off);
    Vec<ES> vu = Ld<ES, LD_PLAIN>::ld(cbyte(up) + off);
    float fd[1], fg[1], fu[1], fh[1], fdg[1], fdu[1];
    Codec<T>::template unpack<ES>(vd, fd);
    Codec<T>::template unpack<ES>(vg, fg);
    Codec<T>::template unpack<ES>(vu, fu);
    Math<FAST, ACT>::bwd_h(fd[0], fg[0], fu[0], c, fh[0], fdg[0], fdu[0]);
    Vec<ES> vh, vdg, vdu;
    Codec<T>::template pack<ES>(fh, vh);
    Codec<T>::template pack<ES>(fdg, vdg);
    Codec<T>::template pack<ES>(fdu, vdu);
    St<ES, ST_PLAIN>::st(byte(h) + off, vh);
    St<ES, ST_PLAIN>::st(byte(dgate) + off, vdg);
    St<ES, ST_PLAIN>::st(byte(dup) + off, vdu);
  }
}

}  // namespace swiglu_b200
