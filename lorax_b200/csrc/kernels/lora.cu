// Multi-adapter LoRA: shrink (v = x A^T) and expand (y += v B^T) over a batch whose tokens may each use a
// different adapter of a different rank, in ONE launch per projection group.
//
// The reference launches one SGMV/BGMV kernel pair per distinct rank in the batch and rebuilds pointer tables on
// the host every step (server/lorax_server/utils/layers.py:114-164, adapters/lora.py:253-396; kernels
// server/punica_kernels/punica_kernels/bgmv/bgmv_impl.cuh:15-192, sgmv_flashinfer/sgmv_flashinfer.cuh:13-353).
// Here the adapter table lives in device memory and changes only when an adapter is loaded or evicted:
//
//   arena      one bf16 allocation that holds every resident adapter
//   slot_base  [S] element offset of the slot's blob inside the arena (< 0: empty slot)
//   slot_rank  [S] padded rank r of the slot (multiple of 8)
//
// Every matrix of an adapter has a size proportional to r, so the blob is laid out as r * (fixed pattern) and a
// matrix is found at  arena + slot_base[s] + r * unit_off  where unit_off depends only on (layer, group).
// Per step the kernels need just tok_slot[T] (slot of each token, -1 = base model), which makes the launch
// shape independent of which adapters or ranks are in the batch (CUDA-graph friendly).
//
// Group layouts:  A_cat [nparts * r, K] (row j = one rank-1 direction, K contiguous)
//                 B_cat [N, r]          (row n = output feature, pre-scaled by alpha / r)
// where the projections fused in one base GEMM (q,k,v or gate,up) are concatenated: output columns
// [0, n0) use rows [0, r) of v, [n0, n1) use [r, 2r), [n1, N) use [2r, 3r).
#include "common.cuh"

namespace lx {

struct LoraTable {
  const __nv_bfloat16* arena;
  const long long* slot_base;
  const int* slot_rank;
  const int* tok_slot;
  int num_slots;
};

LX_DEVICE float dot8(const uint4& a, const uint4& b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  float s = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 fa = unpack_bf16x2(aw[q]), fb = unpack_bf16x2(bw[q]);
    s = fmaf(fa.x, fb.x, s);
    s = fmaf(fa.y, fb.y, s);
  }
  return s;
}

// ------------------------------------------------------------------------------------------------
// shrink
// ------------------------------------------------------------------------------------------------
constexpr int kShrinkKC = 2048;     // K elements staged in shared memory per pass

struct ShrinkParams {
  LoraTable tab;
  const __nv_bfloat16* x;
  long long ldx;
  long long unit_off;
  int nparts;
  float* v;
  int ldv;
  int K, T;
  int* status;
};

// Process TMM consecutive tokens that share `slot`.  xs: [TMM][kShrinkKC] bf16 in shared memory.
template <int TMM, int JW>
LX_DEVICE void shrink_tokens(const ShrinkParams& p, __nv_bfloat16* xs, int t0, int slot, int jbase) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = p.tab.slot_rank[slot];
  const long long base = p.tab.slot_base[slot];
  const int R = r * p.nparts;
  const __nv_bfloat16* A = p.tab.arena + base + (long long)r * p.unit_off;
  float acc[JW][TMM];
#pragma unroll
  for (int a = 0; a < JW; ++a)
#pragma unroll
    for (int m = 0; m < TMM; ++m) acc[a][m] = 0.f;
  const bool any = (base >= 0) && (jbase < R);

  for (int kc0 = 0; kc0 < p.K; kc0 += kShrinkKC) {
    const int kc = min(kShrinkKC, p.K - kc0);
    __syncthreads();
    for (int c = threadIdx.x; c < TMM * (kShrinkKC / 8); c += blockDim.x) {
      const int m = c / (kShrinkKC / 8), e = (c % (kShrinkKC / 8)) * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (e < kc && t0 + m < p.T) val = *reinterpret_cast<const uint4*>(p.x + (long long)(t0 + m) * p.ldx + kc0 + e);
      *reinterpret_cast<uint4*>(xs + m * kShrinkKC + e) = val;
    }
    __syncthreads();
    if (any) {
#pragma unroll
      for (int jl = 0; jl < JW; ++jl) {
        const int j = jbase + warp * JW + jl;
        if (j < R) {
          const __nv_bfloat16* arow = A + (long long)j * p.K + kc0;
#pragma unroll 4
          for (int kk = lane * 8; kk < kc; kk += 256) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(arow + kk));
#pragma unroll
            for (int m = 0; m < TMM; ++m) {
              const uint4 xv = *reinterpret_cast<const uint4*>(xs + m * kShrinkKC + kk);
              acc[jl][m] += dot8(a, xv);
            }
          }
        }
      }
    }
  }
  if (any) {
#pragma unroll
    for (int jl = 0; jl < JW; ++jl) {
      const int j = jbase + warp * JW + jl;
#pragma unroll
      for (int m = 0; m < TMM; ++m) {
        const float s = warp_sum(acc[jl][m]);
        if (lane == 0 && j < R && t0 + m < p.T) p.v[(long long)(t0 + m) * p.ldv + j] = s;
      }
    }
  }
}

template <int TM, int JW>
__global__ void __launch_bounds__(128) lora_shrink_kernel(const ShrinkParams p) {
  extern __shared__ __align__(16) uint8_t lsm[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(lsm);
  const int t0 = blockIdx.x * TM;
  const int jbase = blockIdx.y * 4 * JW;
  int slot0 = p.tab.tok_slot[t0];
  bool uniform = true;
  if (TM > 1) {
#pragma unroll
    for (int m = 1; m < TM; ++m) {
      const int sm = (t0 + m < p.T) ? p.tab.tok_slot[t0 + m] : slot0;
      uniform = uniform && (sm == slot0);
    }
  }
  if (uniform) {
    if (slot0 < 0) return;
    if (slot0 >= p.tab.num_slots) { report_status(p.status, kBadIndex, slot0); return; }
    shrink_tokens<TM, JW>(p, xs, t0, slot0, jbase);
  } else {
    for (int m = 0; m < TM && t0 + m < p.T; ++m) {
      const int s = p.tab.tok_slot[t0 + m];
      if (s < 0) continue;
      if (s >= p.tab.num_slots) { report_status(p.status, kBadIndex, s); continue; }
      shrink_tokens<1, JW>(p, xs, t0 + m, s, jbase);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// expand
// ------------------------------------------------------------------------------------------------
struct ExpandParams {
  LoraTable tab;
  const float* v;
  int ldv;
  long long unit_off;
  __nv_bfloat16* y;
  long long ldy;
  int n0, n1, N, T;
  int* status;
};
constexpr int kExpandMaxR = 3 * 128;

template <int TMM>
LX_DEVICE void expand_tokens(const ExpandParams& p, float* vs, int t0, int slot) {
  const int r = p.tab.slot_rank[slot];
  const long long base = p.tab.slot_base[slot];
  const int n = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  const int nparts_r = (p.n1 < p.N ? 3 : (p.n0 < p.N ? 2 : 1)) * r;
  __syncthreads();
  for (int c = threadIdx.x; c < TMM * nparts_r; c += blockDim.x) {
    const int m = c / nparts_r, j = c % nparts_r;
    vs[m * kExpandMaxR + j] = (t0 + m < p.T) ? p.v[(long long)(t0 + m) * p.ldv + j] : 0.f;
  }
  __syncthreads();
  if (base < 0 || n >= p.N) return;
  const int part = n < p.n0 ? 0 : (n < p.n1 ? 1 : 2);
  const __nv_bfloat16* B = p.tab.arena + base + (long long)r * p.unit_off + (long long)n * r;
  const float* vp = vs + part * r;
  float acc[TMM][2];
#pragma unroll
  for (int m = 0; m < TMM; ++m) acc[m][0] = acc[m][1] = 0.f;
  for (int jc = 0; jc < r; jc += 8) {
    const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(B + jc));
    const uint4 b1 = __ldg(reinterpret_cast<const uint4*>(B + r + jc));
    const uint32_t w0[4] = {b0.x, b0.y, b0.z, b0.w}, w1[4] = {b1.x, b1.y, b1.z, b1.w};
    float f0[8], f1[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = unpack_bf16x2(w0[q]), b = unpack_bf16x2(w1[q]);
      f0[2 * q] = a.x; f0[2 * q + 1] = a.y;
      f1[2 * q] = b.x; f1[2 * q + 1] = b.y;
    }
#pragma unroll
    for (int m = 0; m < TMM; ++m) {
      const float4 va = *reinterpret_cast<const float4*>(vp + m * kExpandMaxR + jc);
      const float4 vb = *reinterpret_cast<const float4*>(vp + m * kExpandMaxR + jc + 4);
      const float vv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        acc[m][0] = fmaf(vv[q], f0[q], acc[m][0]);
        acc[m][1] = fmaf(vv[q], f1[q], acc[m][1]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < TMM; ++m) {
    if (t0 + m < p.T) {
      uint32_t* yp = reinterpret_cast<uint32_t*>(p.y + (long long)(t0 + m) * p.ldy + n);
      const float2 old = unpack_bf16x2(*yp);
      *yp = pack_bf16x2(old.x + acc[m][0], old.y + acc[m][1]);
    }
  }
}

template <int TM>
__global__ void __launch_bounds__(256) lora_expand_kernel(const ExpandParams p) {
  __shared__ __align__(16) float vs[TM * kExpandMaxR];
  const int t0 = blockIdx.x * TM;
  int slot0 = p.tab.tok_slot[t0];
  bool uniform = true;
  if (TM > 1) {
#pragma unroll
    for (int m = 1; m < TM; ++m) {
      const int sm = (t0 + m < p.T) ? p.tab.tok_slot[t0 + m] : slot0;
      uniform = uniform && (sm == slot0);
    }
  }
  if (uniform) {
    if (slot0 < 0) return;
    if (slot0 >= p.tab.num_slots) { report_status(p.status, kBadIndex, slot0); return; }
    expand_tokens<TM>(p, vs, t0, slot0);
  } else {
    for (int m = 0; m < TM && t0 + m < p.T; ++m) {
      const int s = p.tab.tok_slot[t0 + m];
      if (s < 0) continue;
      if (s >= p.tab.num_slots) { report_status(p.status, kBadIndex, s); continue; }
      expand_tokens<1>(p, vs, t0 + m, s);
    }
  }
}

}  // namespace lx

extern "C" {

// v[T, ldv] (fp32) = x[T, K] @ A_cat(slot of token)^T.  Rows of tokens without an adapter are not written.
// max_rank bounds the grid (largest padded rank currently resident).
int lx_lora_shrink(const void* x, long long ldx, const int* tok_slot, const void* arena, const long long* slot_base,
                   const int* slot_rank, int num_slots, long long unit_off, int nparts, float* v, int ldv, int T, int K,
                   int max_rank, int* status, void* stream) {
  using namespace lx;
  if (T <= 0 || max_rank <= 0) return 0;
  if (K % 8 != 0 || ldx % 8 != 0 || nparts * max_rank > ldv) return -1;
  ShrinkParams p{};
  p.tab = LoraTable{reinterpret_cast<const __nv_bfloat16*>(arena), slot_base, slot_rank, tok_slot, num_slots};
  p.x = reinterpret_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.unit_off = unit_off; p.nparts = nparts;
  p.v = v; p.ldv = ldv; p.K = K; p.T = T; p.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int Rmax = nparts * max_rank;
  if (T <= 64) {
    dim3 grid(T, (Rmax + 3) / 4);
    lora_shrink_kernel<1, 1><<<grid, 128, kShrinkKC * 2, s>>>(p);
  } else if (T <= 512) {
    dim3 grid(T, (Rmax + 15) / 16);
    lora_shrink_kernel<1, 4><<<grid, 128, kShrinkKC * 2, s>>>(p);
  } else {
    dim3 grid((T + 7) / 8, (Rmax + 15) / 16);
    lora_shrink_kernel<8, 4><<<grid, 128, 8 * kShrinkKC * 2, s>>>(p);
  }
  return -(int)cudaGetLastError();
}

// y[T, N] (bf16) += v[T, :] @ B_cat(slot of token)^T with the part boundaries n0 <= n1 <= N (all even).
int lx_lora_expand(const float* v, int ldv, const int* tok_slot, const void* arena, const long long* slot_base,
                   const int* slot_rank, int num_slots, long long unit_off, void* y, long long ldy, int T, int N, int n0, int n1,
                   int* status, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if ((N | n0 | n1) & 1 || ldy % 2 != 0) return -1;
  ExpandParams p{};
  p.tab = LoraTable{reinterpret_cast<const __nv_bfloat16*>(arena), slot_base, slot_rank, tok_slot, num_slots};
  p.v = v; p.ldv = ldv; p.unit_off = unit_off;
  p.y = reinterpret_cast<__nv_bfloat16*>(y); p.ldy = ldy; p.n0 = n0; p.n1 = n1; p.N = N; p.T = T; p.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int gy = (N + 511) / 512;
  if (T <= 512) {
    dim3 grid(T, gy);
    lora_expand_kernel<1><<<grid, 256, 0, s>>>(p);
  } else {
    dim3 grid((T + 7) / 8, gy);
    lora_expand_kernel<8><<<grid, 256, 0, s>>>(p);
  }
  return -(int)cudaGetLastError();
}

}  // extern "C"
