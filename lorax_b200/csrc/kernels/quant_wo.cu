// Weight-only group quantisation (GPTQ / AWQ / EETQ / bitsandbytes / HQQ checkpoints after repacking): the weights stay
// packed in HBM and are expanded to bf16 on the way to the tensor cores.
//
// One resident format serves every source format (lorax_b200/utils/quant_formats.py does the repacking):
//   codes   uint8 [N, K * bits / 8]   bits in {2, 4, 8}; code j of a byte sits at bit j * bits.  For 4 bits the eight codes
//                                     of a 32-bit word are interleaved: nibble i holds k = 8 * word + {0,2,4,6,1,3,5,7}[i],
//                                     so that (nibble i, nibble i + 4) is a pair of neighbouring k and one mask yields a
//                                     ready bf16x2 operand
//   sz      half2 [N, K / group]      (scale, zero): w = (code - zero) * scale; zero may be fractional (HQQ)
//   table   float [16] or null        code book formats (nf4 / fp4): w = table[code] * scale
//
// Two kernels:
//   wq_dequant_kernel   packed -> bf16 [N, K] (any bits, code book or affine).  Used in front of the tcgen05 GEMM when a
//                       step has many tokens (the GEMM is compute bound there and the expansion is a small extra).
//   wq4_mma_kernel      out[T, N] = x[T, K] . W^T for T <= 32 straight from the 4-bit codes: every warp streams 16 or 32
//                       weight rows, expands 32 codes per lane and row in registers (one lop3 + one subtract + one fma per pair)
//                       and feeds them to m16n8k16 tensor-core MMAs as the A operand; tokens are the N side.  The K
//                       range is split over the 8 warps of a block and summed through shared memory.  HBM traffic is the
//                       packed weights once: a quarter of the bf16 GEMM's at decode sizes.
//
// The reference serves these formats with exllama / exllamav2 (server/exllama_kernels, server/exllamav2_kernels), the AWQ
// and EETQ extensions (server/lorax_server/utils/awq/awq.py:39, layers/eetq.py:2-25), bitsandbytes (layers/bnb.py), HQQ
// (layers/hqq.py) and a Triton kernel (layers/gptq/quant_linear.py:106-230).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace lx {

struct WqDequantParams {
  const uint8_t* codes;
  const __half2* sz;
  const float* table;
  __nv_bfloat16* out;
  long long ldo;
  int N, K, bits, group;
};

// One thread expands 16 bytes of codes (128 / bits consecutive k of one row, all inside one group).
__global__ void __launch_bounds__(256) wq_dequant_kernel(const WqDequantParams p) {
  const int vpc = 128 / p.bits;                       // values per 16-byte chunk
  const int chunks_per_row = p.K / vpc;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)p.N * chunks_per_row) return;
  const int n = (int)(idx / chunks_per_row), c = (int)(idx % chunks_per_row);
  const int k0 = c * vpc;
  const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p.codes + (long long)n * (p.K * p.bits / 8) + (long long)c * 16));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  const __half2 szv = p.sz[(long long)n * (p.K / p.group) + k0 / p.group];
  const float s = __low2float(szv), z = __high2float(szv);
  __nv_bfloat16* dst = p.out + (long long)n * p.ldo + k0;
  float tab[16];
  if (p.table != nullptr) {
#pragma unroll
    for (int i = 0; i < 16; ++i) tab[i] = p.table[i];
  }
  if (p.bits == 4) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {                   // pair j = k offsets (2j, 2j + 1) = nibbles (j, j + 4)
        const int c0 = (w[q] >> (4 * j)) & 15, c1 = (w[q] >> (4 * j + 16)) & 15;
        float f0, f1;
        if (p.table != nullptr) { f0 = tab[c0] * s; f1 = tab[c1] * s; }
        else { f0 = ((float)c0 - z) * s; f1 = ((float)c1 - z) * s; }
        o[j] = pack_bf16x2(f0, f1);
      }
      *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else if (p.bits == 8) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t word = w[2 * q + (j >> 1)];
        const int c0 = (word >> (16 * (j & 1))) & 255, c1 = (word >> (16 * (j & 1) + 8)) & 255;
        o[j] = pack_bf16x2(((float)c0 - z) * s, ((float)c1 - z) * s);
      }
      *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {                                            // 2 bits: 64 values
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      uint32_t o[4];
      const uint32_t half16 = (w[q >> 1] >> (16 * (q & 1))) & 0xffffu;      // 8 codes
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = (half16 >> (4 * j)) & 3, c1 = (half16 >> (4 * j + 2)) & 3;
        o[j] = pack_bf16x2(((float)c0 - z) * s, ((float)c1 - z) * s);
      }
      *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ 4-bit tensor-core GEMM, few tokens

constexpr int kWqWarps = 8;
constexpr int kWqRows = 16;                           // weight rows per block (the M of m16n8k16)

struct Wq4Params {
  const uint8_t* codes;
  const __half2* sz;
  const __nv_bfloat16* x;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  long long ldx, ldo;
  int T, N, K, group;
};

LX_DEVICE void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four bf16x2 operands (k pairs 01, 23, 45, 67) from one word of interleaved 4-bit codes.  0x4300 is bf16 128.0 with an ulp of 1,
// so or-ing a nibble into the mantissa gives 128 + code exactly; the subtraction of 128 + round(zero) is exact as well.
LX_DEVICE void wq4_expand(uint32_t w, __nv_bfloat162 bias128z, __nv_bfloat162 s2, __nv_bfloat162 c2, uint32_t (&o)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v = ((w >> (4 * j)) & 0x000f000fu) | 0x43004300u;
    __nv_bfloat162 f = *reinterpret_cast<__nv_bfloat162*>(&v);
    f = __hfma2(__hsub2(f, bias128z), s2, c2);
    o[j] = *reinterpret_cast<uint32_t*>(&f);
  }
}

// The same without the scale: (code - zero) as exact small integers.
LX_DEVICE void wq4_expand_int(uint32_t w, __nv_bfloat162 bias128z, uint32_t (&o)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v = ((w >> (4 * j)) & 0x000f000fu) | 0x43004300u;
    __nv_bfloat162 f = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias128z);
    o[j] = *reinterpret_cast<uint32_t*>(&f);
  }
}

struct Wq4Group {
  __nv_bfloat162 bias128z, s2, c2;
};
LX_DEVICE Wq4Group wq4_group(__half2 szv) {
  const float s = __low2float(szv), z = __high2float(szv);
  const float zi = rintf(z);
  Wq4Group g;
  g.bias128z = __float2bfloat162_rn(128.f + zi);
  g.s2 = __float2bfloat162_rn(s);
  g.c2 = __float2bfloat162_rn((zi - z) * s);          // fractional part of the zero point, |.| <= s / 2
  return g;
}

// Every warp owns the k-blocks warp, warp + 8, ... of the block's 16 * MT weight rows; the next k-block's codes are in flight
// while the current one is multiplied.  One activation fragment feeds MT row tiles.
// EXACT: every 128-wide k-block lies inside one group and the zero points are integers.  The codes then go to the tensor cores as
// the exact integers (code - zero); the k-block's partial product is scaled by the group's fp16 scale in fp32 on its way into the
// accumulator: no fma per pair of weights and no bf16 rounding of the scale.
template <int NT, int MT, bool EXACT>                  // token tiles of 8, row tiles of 16
__global__ void __launch_bounds__(kWqWarps * 32, 2) wq4_mma_kernel(const Wq4Params p) {
  __shared__ float red[kWqWarps][kWqRows * MT][8 * NT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * kWqRows * MT;
  const int G = p.K / p.group;
  const long long row_bytes = p.K / 2;
  const uint8_t* c_r0 = p.codes + (long long)(n0 + g) * row_bytes + 16 * t;           // row tile m adds 16 rows
  const __half2* sz_r0 = p.sz + (long long)(n0 + g) * G;
  float acc[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f;

  const int kblocks = p.K / 128;
  uint4 nc0[MT], nc1[MT];
  __half2 nsz0[MT], nsz1[MT];
  auto fetch = [&](int kb) {
    const int grp = (kb * 128 + 32 * t) / p.group;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      nc0[m] = __ldcs(reinterpret_cast<const uint4*>(c_r0 + (16 * m) * row_bytes + (long long)kb * 64));
      nc1[m] = __ldcs(reinterpret_cast<const uint4*>(c_r0 + (16 * m + 8) * row_bytes + (long long)kb * 64));
      nsz0[m] = sz_r0[(long long)(16 * m) * G + grp];
      nsz1[m] = sz_r0[(long long)(16 * m + 8) * G + grp];
    }
  };
  int kb = warp;
  if (kb < kblocks) fetch(kb);
  for (; kb < kblocks; kb += kWqWarps) {
    uint32_t a0[MT][4][4], a1[MT][4][4];               // [row tile][word][pair]: rows g and g + 8
    float s0[MT], s1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if constexpr (EXACT) {
        s0[m] = __low2float(nsz0[m]);
        s1[m] = __low2float(nsz1[m]);
        const __nv_bfloat162 z0 = __float2bfloat162_rn(128.f + __high2float(nsz0[m])), z1 = __float2bfloat162_rn(128.f + __high2float(nsz1[m]));
        wq4_expand_int(nc0[m].x, z0, a0[m][0]);
        wq4_expand_int(nc0[m].y, z0, a0[m][1]);
        wq4_expand_int(nc0[m].z, z0, a0[m][2]);
        wq4_expand_int(nc0[m].w, z0, a0[m][3]);
        wq4_expand_int(nc1[m].x, z1, a1[m][0]);
        wq4_expand_int(nc1[m].y, z1, a1[m][1]);
        wq4_expand_int(nc1[m].z, z1, a1[m][2]);
        wq4_expand_int(nc1[m].w, z1, a1[m][3]);
        continue;
      }
      const Wq4Group g0 = wq4_group(nsz0[m]), g1 = wq4_group(nsz1[m]);
      wq4_expand(nc0[m].x, g0.bias128z, g0.s2, g0.c2, a0[m][0]);
      wq4_expand(nc0[m].y, g0.bias128z, g0.s2, g0.c2, a0[m][1]);
      wq4_expand(nc0[m].z, g0.bias128z, g0.s2, g0.c2, a0[m][2]);
      wq4_expand(nc0[m].w, g0.bias128z, g0.s2, g0.c2, a0[m][3]);
      wq4_expand(nc1[m].x, g1.bias128z, g1.s2, g1.c2, a1[m][0]);
      wq4_expand(nc1[m].y, g1.bias128z, g1.s2, g1.c2, a1[m][1]);
      wq4_expand(nc1[m].z, g1.bias128z, g1.s2, g1.c2, a1[m][2]);
      wq4_expand(nc1[m].w, g1.bias128z, g1.s2, g1.c2, a1[m][3]);
    }
    if (kb + kWqWarps < kblocks) fetch(kb + kWqWarps); // next block's codes are in flight while this one is multiplied
    const long long kx = (long long)kb * 128 + 32 * t;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int tok = 8 * j + g;
      uint4 xv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        xv[q] = tok < p.T ? __ldg(reinterpret_cast<const uint4*>(p.x + tok * p.ldx + kx + 8 * q)) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float part[4] = {0.f, 0.f, 0.f, 0.f};
        float (&dst)[4] = EXACT ? part : acc[m][j];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // the k order inside an MMA is (pair 0 | pair 1) resp. (pair 2 | pair 3) of this lane's word: the same for A and B
          mma_bf16_16816(dst, a0[m][q][0], a1[m][q][0], a0[m][q][1], a1[m][q][1], xv[q].x, xv[q].y);
          mma_bf16_16816(dst, a0[m][q][2], a1[m][q][2], a0[m][q][3], a1[m][q][3], xv[q].z, xv[q].w);
        }
        if constexpr (EXACT) {                         // rows g (c0, c1) and g + 8 (c2, c3) have their own scales
          acc[m][j][0] = fmaf(s0[m], part[0], acc[m][j][0]);
          acc[m][j][1] = fmaf(s0[m], part[1], acc[m][j][1]);
          acc[m][j][2] = fmaf(s1[m], part[2], acc[m][j][2]);
          acc[m][j][3] = fmaf(s1[m], part[3], acc[m][j][3]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      red[warp][16 * m + g][8 * j + 2 * t] = acc[m][j][0];
      red[warp][16 * m + g][8 * j + 2 * t + 1] = acc[m][j][1];
      red[warp][16 * m + g + 8][8 * j + 2 * t] = acc[m][j][2];
      red[warp][16 * m + g + 8][8 * j + 2 * t + 1] = acc[m][j][3];
    }
  }
  __syncthreads();
  constexpr int kRows = kWqRows * MT;
  for (int o = threadIdx.x; o < kRows * 8 * NT; o += kWqWarps * 32) {
    const int tok = o / kRows, r = o % kRows;          // neighbouring threads write neighbouring features of one token
    if (tok < p.T) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kWqWarps; ++w) v += red[w][r][tok];
      if (p.bias != nullptr) v += __bfloat162float(p.bias[n0 + r]);
      p.out[tok * p.ldo + n0 + r] = __float2bfloat16(v);
    }
  }
}

template <int NT, int MT>
int wq4_launch(const Wq4Params& p, bool exact, cudaStream_t s) {
  if (exact) wq4_mma_kernel<NT, MT, true><<<p.N / (kWqRows * MT), kWqWarps * 32, 0, s>>>(p);
  else wq4_mma_kernel<NT, MT, false><<<p.N / (kWqRows * MT), kWqWarps * 32, 0, s>>>(p);
  return -(int)cudaGetLastError();
}

}  // namespace lx

extern "C" {

// Packed weights -> bf16 [N, K] (row stride ldo elements).  bits in {2, 4, 8}; `table` (16 floats on the device) selects the
// code book form for 4 bits.  K * bits must be a multiple of 128 and a 16-byte chunk must not straddle a group.
int lx_wq_dequant(const void* codes, const void* sz, const void* table, void* out, long long ldo, int N, int K, int bits, int group,
                  void* stream) {
  using namespace lx;
  if (bits != 2 && bits != 4 && bits != 8) return -1;
  const int vpc = 128 / bits;
  if (N <= 0 || K <= 0 || K % vpc != 0 || group % vpc != 0 || K % group != 0 || ldo % 8 != 0) return -1;
  if (table != nullptr && bits != 4) return -1;
  WqDequantParams p{static_cast<const uint8_t*>(codes), static_cast<const __half2*>(sz), static_cast<const float*>(table),
                    static_cast<__nv_bfloat16*>(out), ldo, N, K, bits, group};
  const long long chunks = (long long)N * (K / vpc);
  wq_dequant_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return -(int)cudaGetLastError();
}

int lx_wq4_max_tokens() { return 32; }

// out[T, N] = x[T, K] . W^T (+ bias) for T <= 32 from affine 4-bit codes.  N % 16 == 0, K % 128 == 0, group % 32 == 0, x rows
// 16-byte aligned.
int lx_wq4_gemm_ex(const void* x, long long ldx, const void* codes, const void* sz, const void* bias, void* out, long long ldo, int T, int N,
                   int K, int group, int integer_zeros, void* stream);

int lx_wq4_gemm(const void* x, long long ldx, const void* codes, const void* sz, const void* bias, void* out, long long ldo, int T, int N,
                int K, int group, void* stream) {
  return lx_wq4_gemm_ex(x, ldx, codes, sz, bias, out, ldo, T, N, K, group, 0, stream);
}

// `integer_zeros` != 0 promises that every zero point is an integer (GPTQ, AWQ, round-to-nearest; not HQQ): with groups that are
// multiples of 128 the kernel then multiplies exact integers and scales the partial sums (see EXACT above).
int lx_wq4_gemm_ex(const void* x, long long ldx, const void* codes, const void* sz, const void* bias, void* out, long long ldo, int T, int N,
                   int K, int group, int integer_zeros, void* stream) {
  using namespace lx;
  if (T <= 0 || T > 32 || N % kWqRows != 0 || K % 128 != 0 || group % 32 != 0 || K % group != 0 || ldx % 8 != 0) return -1;
  Wq4Params p{static_cast<const uint8_t*>(codes), static_cast<const __half2*>(sz), static_cast<const __nv_bfloat16*>(x),
              static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(out), ldx, ldo, T, N, K, group};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // two row tiles per warp halve the re-reads of the activations (every block reads all of x); with few rows and few tokens
  // the larger grid of single tiles fills the machine better
  const bool two = N % (2 * kWqRows) == 0 && (N >= 8192 || T > 8);
  // measured: the exact-integer path wins 6-15 % on the large projections at up to 8 tokens and loses elsewhere (register
  // pressure with two token tiles; small grids)
  const bool exact = integer_zeros != 0 && group % 128 == 0 && T <= 8 && (N >= 16384 || K >= 8192);
  if (T <= 8) return two ? wq4_launch<1, 2>(p, exact, s) : wq4_launch<1, 1>(p, exact, s);
  if (T <= 16) return two ? wq4_launch<2, 2>(p, exact, s) : wq4_launch<2, 1>(p, exact, s);
  return wq4_launch<4, 1>(p, exact, s);
}

}  // extern "C"
