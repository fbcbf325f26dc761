// Block-scaled fp8 (e4m3) GEMM on the 5th-generation tensor cores.
//
//   out[t, n] = sum_kb  sa[kb, t] * sw[n / 128, kb] * sum_{k in block kb} xq[t, k] * wq[n, k]     (+ bias[n])
//
// Weights are quantised offline in 128 x 128 blocks (one fp32 scale per block), activations on the fly per token and
// 128-wide K block (one fp32 scale per 1 x 128 strip).  The reference serves fp8 checkpoints through per-tensor
// scaled `torch._scaled_mm` / vLLM kernels (server/lorax_server/layers/fp8.py:1-60); the 128 x 128 scheme keeps
// outlier blocks from costing the whole tensor its mantissa.
//
// The scales change every 128 elements of K, so products cannot simply keep accumulating in TMEM.  One pipeline
// stage is exactly one scale block (128 fp8 = one 128-byte swizzle row): the MMA warp issues four
// tcgen05.mma.kind::f8f6f4 (K = 32 each) into one of two TMEM accumulators with accumulate = 0 on the first, commits,
// and moves on to the other accumulator; eight epilogue warps (two per TMEM lane quadrant, half of the columns each) pull
// the finished 128 x bn partial out of TMEM with
// tcgen05.ld, multiply by the block's scales and add into fp32 registers while the tensor core already works on the
// next block.  Weights take the UMMA M side (128 output features per tile, so a tile sees one weight scale per K
// block), tokens the N side in tiles of up to 128.
#include <cuda_fp8.h>

#include "common.cuh"

namespace lx {

constexpr int kF8BM = 128;
constexpr int kF8BK = 128;          // fp8 elements per stage = bytes per swizzle row = one scale block
constexpr int kF8EpiWarps = 8;       // two per TMEM lane quadrant, each takes half of the tile's columns
constexpr int kF8Threads = 64 + 32 * kF8EpiWarps;

struct Fp8Params {
  int N, T, K;
  int bn;                       // token tile (multiple of 16, <= BN)
  const float* sw;              // [ceil(N/128)][kblocks] weight block scales
  const float* sa;              // [kblocks][ld_sa] activation scales (transposed: tokens contiguous)
  int ld_sa;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;
  int ksplit;                   // > 1: every tile's K range is cut into ksplit parts, each writes fp32 to `partial`
  float* partial;               // [ksplit][T][N]
  int* status;
};

template <int BN, int STAGES>
struct Fp8Smem {
  static constexpr int kABytes = kF8BM * kF8BK;
  static constexpr int kBBytes = BN * kF8BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kScaleBytes = 2 * BN * 4;
  static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + kScaleBytes + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_block128_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const Fp8Params p) {
  using S = Fp8Smem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  float* scale_stage = reinterpret_cast<float*>(smem + STAGES * S::kStageBytes + S::kBarrierBytes);   // [2][BN]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  const int tiles_a = (p.N + kF8BM - 1) / kF8BM;
  const int tiles_b = (p.T + p.bn - 1) / p.bn;
  const int num_tiles = tiles_a * tiles_b;
  const int kblocks = (p.K + kF8BK - 1) / kF8BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tmem_full[s], 1); mbar_init(&tmem_empty[s], kF8EpiWarps); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) { tmem_alloc(tmem_base_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_tiles * p.ksplit && ok; w += gridDim.x) {
        const int tile = w / p.ksplit, split = w % p.ksplit;
        const int ta = tile / tiles_b, tb = tile % tiles_b;    // token tiles of one weight tile run side by side
        const int kb0 = (int)((long long)kblocks * split / p.ksplit), kb1 = (int)((long long)kblocks * (split + 1) / p.ksplit);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { report_status(p.status, kTimeoutEmptyBarrier, w); *abort_flag = 1; ok = false; break; }
          uint8_t* sa = smem + stage * S::kStageBytes;
          mbar_expect_tx(&full_bar[stage], (uint32_t)(S::kABytes + p.bn * kF8BK));
          tma_load_2d_hint(sa, &tmap_w, &full_bar[stage], kb * kF8BK, ta * kF8BM, pol_w);
          tma_load_2d_hint(sa + S::kABytes, &tmap_x, &full_bar[stage], kb * kF8BK, tb * p.bn, pol_x);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kF8BM, (uint32_t)p.bn, kFmtE4M3, kFmtE4M3);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      for (int w = blockIdx.x; w < num_tiles * p.ksplit && ok; w += gridDim.x) {
        const int split = w % p.ksplit;
        const int kb0 = (int)((long long)kblocks * split / p.ksplit), kb1 = (int)((long long)kblocks * (split + 1) / p.ksplit);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1, abort_flag)) { report_status(p.status, kTimeoutTmemEmpty, w); *abort_flag = 1; ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { report_status(p.status, kTimeoutFullBarrier, w); *abort_flag = 1; ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint64_t da = make_desc_k_sw128(sa), db = make_desc_k_sw128(sa + S::kABytes);
          const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
#pragma unroll
          for (int k = 0; k < kF8BK / 32; ++k) umma_f8f6f4_ss(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k > 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          tc_commit(&tmem_full[acc]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          acc_phase[acc] ^= 1;
          acc ^= 1;
        }
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                // which half of the tile's columns this warp accumulates
    const int row_in_tile = quad * 32 + lane;
    const int te = threadIdx.x - 64;                 // 0..255 among the epilogue threads
    constexpr int HB = BN / 2;                       // columns per thread
    const int c_lo = half * HB;
    int acc = 0; uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    for (int w = blockIdx.x; w < num_tiles * p.ksplit && ok; w += gridDim.x) {
      const int tile = w / p.ksplit, split = w % p.ksplit;
      const int ta = tile / tiles_b, tb = tile % tiles_b;
      const int kb0 = (int)((long long)kblocks * split / p.ksplit), kb1 = (int)((long long)kblocks * (split + 1) / p.ksplit);
      const int n = ta * kF8BM + row_in_tile;
      const int t0 = tb * p.bn;
      float sum[HB];
#pragma unroll
      for (int q = 0; q < HB; ++q) sum[q] = 0.f;
      // the scales of a K block are fetched one block ahead: their trip to L2 must not sit between two MMAs
      const bool stager = te < p.bn && t0 + te < p.T;
      float next_scale = 0.f;
      if (stager && kb0 < kb1) next_scale = p.sa[(long long)kb0 * p.ld_sa + t0 + te] * p.sw[(long long)ta * kblocks + kb0];
      for (int kb = kb0; kb < kb1; ++kb) {
        float* sc = scale_stage + acc * BN;
        if (te < p.bn) sc[te] = next_scale;
        if (stager && kb + 1 < kb1) next_scale = p.sa[(long long)(kb + 1) * p.ld_sa + t0 + te] * p.sw[(long long)ta * kblocks + kb + 1];
        if (!mbar_wait(&tmem_full[acc], acc_phase[acc], abort_flag)) { report_status(p.status, kTimeoutTmemFull, w); *abort_flag = 1; ok = false; }
        // every epilogue thread reaches the barrier, also after a time-out, so that nobody is left waiting at it
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kF8EpiWarps) : "memory");
        if (*abort_flag) { ok = false; break; }
        tc_fence_after();
        acc_phase[acc] ^= 1;
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c_lo);
        constexpr int CH = HB >= 32 ? 32 : 16;
#pragma unroll
        for (int c = 0; c < HB; c += CH) {
          if (c_lo + c < p.bn) {
            uint32_t r[CH];
            if constexpr (CH == 32) tmem_ld_32x32b_x32(taddr + c, r); else tmem_ld_32x32b_x16(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < CH; q += 4) {
              const float4 s4 = *reinterpret_cast<const float4*>(sc + c_lo + c + q);
              sum[c + q] = fmaf(__uint_as_float(r[q]), s4.x, sum[c + q]);
              sum[c + q + 1] = fmaf(__uint_as_float(r[q + 1]), s4.y, sum[c + q + 1]);
              sum[c + q + 2] = fmaf(__uint_as_float(r[q + 2]), s4.z, sum[c + q + 2]);
              sum[c + q + 3] = fmaf(__uint_as_float(r[q + 3]), s4.w, sum[c + q + 3]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        acc ^= 1;
      }
      if (!ok) break;
      if (n < p.N) {
        if (p.ksplit > 1) {
          float* dst = p.partial + ((long long)split * p.T + t0 + c_lo) * p.N + n;
#pragma unroll
          for (int q = 0; q < HB; ++q) {
            if (c_lo + q < p.bn && t0 + c_lo + q < p.T) __stcg(dst + (long long)q * p.N, sum[q]);
          }
        } else {
          const float b = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
          for (int q = 0; q < HB; ++q) {
            if (c_lo + q < p.bn && t0 + c_lo + q < p.T) p.out[(long long)(t0 + c_lo + q) * p.ldo + n] = __float2bfloat16(sum[q] + b);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

// x[T, K] bf16 -> xq[T, K] e4m3 and sa[kb, t] = amax(x[t, block kb]) / 448.  One warp per (token, K block).
__global__ void __launch_bounds__(256) quant_act_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ xq,
                                                            long long ldq, float* __restrict__ sa, int ld_sa, int T, int K) {
  const int kblocks = (K + 127) / 128;
  const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= (long long)T * kblocks) return;
  const int t = (int)(item / kblocks), kb = (int)(item % kblocks);
  const int lane = threadIdx.x & 31;
  const int k = kb * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (k + 3 < K) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + (long long)t * ldx + k);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int q = 0; q < 4; ++q) if (k + q < K) v[q] = __bfloat162float(x[(long long)t * ldx + k + q]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.f;
  const float inv = 1.f / scale;
  if (lane == 0) sa[(long long)kb * ld_sa + t] = scale;
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
  if (k + 3 < K) {
    *reinterpret_cast<uint32_t*>(xq + (long long)t * ldq + k) = (uint32_t)lo | ((uint32_t)hi << 16);
  } else {
    const uint32_t pk = (uint32_t)lo | ((uint32_t)hi << 16);
    for (int q = 0; q < 4; ++q) if (k + q < K) xq[(long long)t * ldq + k + q] = (uint8_t)(pk >> (8 * q));
  }
}

// out[t, n] = bf16(sum_s partial[s, t, n] + bias[n]): the K splits in split order.
__global__ void __launch_bounds__(256) fp8_splitk_reduce_kernel(const float* __restrict__ partial, int ksplit, int T, int N,
                                                                const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, long long ldo) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= (long long)T * N) return;
  const int t = (int)(i / N), n = (int)(i % N);
  float a = 0.f;
  for (int s = 0; s < ksplit; ++s) a += __ldcg(partial + ((long long)s * T + t) * N + n);
  if (bias != nullptr) a += __bfloat162float(bias[n]);
  out[(long long)t * ldo + n] = __float2bfloat16(a);
}

typedef CUresult (*EncodeTiledFn3)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn3 encode_fn3() {
  static EncodeTiledFn3 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn3>(ptr);
  }
  return fn;
}

// 2-D K-major byte tensor map: dims {K, rows}, box {128, box_rows}, 128-byte swizzle, zero fill outside.
static int make_tmap_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t K, uint64_t row_stride_bytes, uint32_t box_rows) {
  EncodeTiledFn3 fn = encode_fn3();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {(cuuint32_t)kF8BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

template <int BN, int STAGES>
static int launch_fp8(const CUtensorMap& tw, const CUtensorMap& tx, const Fp8Params& p, int grid, cudaStream_t stream) {
  using S = Fp8Smem<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_block128_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  gemm_fp8_block128_kernel<BN, STAGES><<<grid, kF8Threads, S::kTotal, stream>>>(tw, tx, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace lx

extern "C" {

// xq / sa from x (see quant_act_fp8_kernel).  K and the row strides must be multiples of 16 for the TMA that follows.
int lx_quant_act_fp8(const void* x, long long ldx, void* xq, long long ldq, float* sa, int ld_sa, int T, int K, void* stream) {
  if (T <= 0) return 0;
  if (K % 4 != 0 || ldx % 4 != 0 || ldq % 4 != 0) return -1;
  const long long items = (long long)T * ((K + 127) / 128);
  lx::quant_act_fp8_kernel<<<(unsigned)((items + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<uint8_t*>(xq), ldq, sa, ld_sa, T, K);
  return -(int)cudaGetLastError();
}

// out[T, N] (bf16) = block-scaled fp8 product of xq[T, K] (scales sa[kb, t]) and wq[N, K] (scales sw[N/128, K/128]) + bias.
int lx_gemm_fp8_block128(const void* xq, long long ldq, const float* sa, int ld_sa, const void* wq, long long ldw, const float* sw,
                         void* out, long long ldo, const void* bias, int T, int N, int K, void* ws, long long ws_bytes, int* status,
                         int num_sms, void* stream_) {
  using namespace lx;
  if (T <= 0 || N <= 0) return 0;
  if (K % 16 != 0 || ldq % 16 != 0 || ldw % 16 != 0) return -1000;
  Fp8Params p{};
  p.N = N; p.T = T; p.K = K;
  p.sw = sw; p.sa = sa; p.ld_sa = ld_sa;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  // token tile: the fewest tiles of at most 128 tokens, evenly sized
  const int t16 = (T + 15) / 16 * 16;
  const int ttiles = (t16 + 127) / 128;
  int bn = ((t16 + ttiles - 1) / ttiles + 15) / 16 * 16;
  if (bn > 128) bn = 128;
  p.bn = bn;
  CUtensorMap tw, tx;
  if (make_tmap_u8(&tw, wq, N, K, ldw, kF8BM)) return -1002;
  if (make_tmap_u8(&tx, xq, T, K, ldq, bn)) return -1003;
  const int tiles = ((N + kF8BM - 1) / kF8BM) * ((T + bn - 1) / bn);
  // few tiles (decode, narrow projections): cut K so that every SM streams weights; a second small kernel adds the parts
  const int kblocks = (K + kF8BK - 1) / kF8BK;
  int ks = 1;
  while (tiles * (ks + 1) <= num_sms && kblocks / (ks + 1) >= 4 && ks < 8 && ws != nullptr &&
         (long long)(ks + 1) * T * N * 4 <= ws_bytes) ++ks;
  p.ksplit = ks;
  p.partial = reinterpret_cast<float*>(ws);
  const int work = tiles * ks;
  const int grid = work < num_sms ? work : num_sms;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int rc;
  if (bn <= 32) rc = launch_fp8<32, 8>(tw, tx, p, grid, stream);
  else if (bn <= 64) rc = launch_fp8<64, 8>(tw, tx, p, grid, stream);
  else rc = launch_fp8<128, 6>(tw, tx, p, grid, stream);
  if (rc != 0 || ks == 1) return rc;
  const long long total = (long long)T * N;
  fp8_splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(p.partial, ks, T, N, p.bias, p.out, ldo);
  return -(int)cudaGetLastError();
}

}  // extern "C"


// ------------------------------------------------------------------------------------------------
// Block-scaled e4m3 weights -> bf16, one pass.  For long prefills the fp8 GEMM above is bound by the per-128 promotion of its
// partial sums; expanding a projection's weights (about 0.1 ms for a 7B-class layer) and running the bf16 GEMM on them is more
// than twice as fast from a few hundred rows on, and the activations keep their bf16 precision.  The weights stay fp8 in
// memory; the scratch holds one projection at a time.
// ------------------------------------------------------------------------------------------------
namespace lx {

__global__ void __launch_bounds__(256) fp8_block128_dequant_kernel(const uint8_t* __restrict__ q, long long ldq, const float* __restrict__ sw,
                                                                   int lds, __nv_bfloat16* __restrict__ out, long long ldo, int N, int K) {
  pdl_wait();
  const long long vecs_per_row = K / 16;
  const long long total = (long long)N * vecs_per_row;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(v / vecs_per_row), k = (int)(v % vecs_per_row) * 16;
    const float sc = sw[(n >> 7) * lds + (k >> 7)];
    const uint4 raw = *reinterpret_cast<const uint4*>(q + (long long)n * ldq + k);
    const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_fp8x2_storage_t pair = (__nv_fp8x2_storage_t)((w4[i] >> (16 * h)) & 0xffffu);
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        o[2 * i + h] = pack_bf16x2(f.x * sc, f.y * sc);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + (long long)n * ldo + k);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace lx

extern "C" {

// out[N, K] (bf16) = e4m3(q[N, K]) * scale[n / 128][k / 128]; K a multiple of 16, 16-byte aligned rows.
int lx_fp8_block128_dequant(const void* q, long long ldq, const float* sw, int lds, void* out, long long ldo, int N, int K, void* stream) {
  using namespace lx;
  if (N <= 0 || K <= 0) return 0;
  if (K % 16 != 0 || ldq % 16 != 0 || ldo % 8 != 0) return -1;
  const long long total = (long long)N * (K / 16);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  launch_pdl(fp8_block128_dequant_kernel, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
             reinterpret_cast<const uint8_t*>(q), ldq, sw, lds, reinterpret_cast<__nv_bfloat16*>(out), ldo, N, K);
  return -(int)cudaGetLastError();
}

}  // extern "C"
