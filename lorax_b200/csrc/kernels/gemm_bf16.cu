// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands fed by TMA).
//
//   out[i, j] = sum_k A[i, k] * B[j, k]  (+ bias)          A: [a_rows, K]   B: [b_rows, K]   both K-contiguous
//
// One kernel serves every dense projection of the decoder (QKV, O, gate_up, down, lm_head), which the
// reference computes with cuBLAS through `torch.nn.functional.linear` (server/lorax_server/layers/linear.py:38).
// Both operands are "K-major", which is how activations [tokens, K] and nn.Linear weights [N, K] already sit in
// memory, so either can take the UMMA M side:
//   * prefill (many tokens):  A = activations, B = weights, 128 x 256 tiles, compute bound;
//   * decode (few tokens):    A = weights (128 output features per tile), B = activations (UMMA N = tokens
//     rounded up to 16), so the tensor core does no work for padding rows and each weight byte is read from
//     HBM exactly once.  Small grids are widened with split-K; the last CTA to finish a tile reduces the
//     fp32 partials in a fixed order (deterministic) and writes bf16.
//
// Structure: persistent CTAs of 6 warps.  Warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) and
// TMEM owner, warps 2..5 = epilogue (each warp reads its own 32-lane TMEM quadrant with tcgen05.ld).  A STAGES
// deep smem ring is guarded by full/empty mbarriers; the accumulator is double buffered in TMEM so the epilogue
// of tile i overlaps the main loop of tile i+1.
#include "common.cuh"

namespace lx {

constexpr int kBM = 128;   // UMMA M (rows of operand A per tile)
constexpr int kBK = 64;    // K per pipeline stage: 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr int lx_gemm_max_tiles_const = 8192;

struct GemmParams {
  int a_rows, b_rows, K;
  int umma_n;                 // runtime UMMA N (multiple of 16, <= BN)
  __nv_bfloat16* out;
  long long ldo_a, ldo_b;     // out[i * ldo_a + j * ldo_b]
  const __nv_bfloat16* bias;  // optional, indexed by the feature dimension
  int bias_on_a;              // 1: bias[i] (weights are operand A), 0: bias[j]
  int split_k;
  float* ws;                  // split-K partials: [tile][split][128][BN] fp32
  int* counters;              // split-K arrival counters, one per tile, zero between launches
  int* status;                // [2] status word + detail
  int hint_a_first;           // 1: operand A is streamed once (weights) -> evict_first, B evict_last; 0: opposite
  float out_scale;            // multiplies the accumulator (logit scaling); 1.0 normally
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + 1024;  // +1024 for manual alignment
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int* last_flag = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_base_slot + 2));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;

  const int tiles_a = (p.a_rows + kBM - 1) / kBM;
  const int tiles_b = (p.b_rows + BN - 1) / BN;
  const int num_tiles = tiles_a * tiles_b;
  const int num_work = num_tiles * p.split_k;
  const int kblocks = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], 4);
    }
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  // Work item w -> (tile, split).  Tiles are ordered with the A tile index fastest inside one B tile so that
  // CTAs running at the same time share the B operand through L2.
  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_a = p.hint_a_first ? policy_evict_first() : policy_evict_last();
      const uint64_t pol_b = p.hint_a_first ? policy_evict_last() : policy_evict_first();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int tile = w / p.split_k, split = w % p.split_k;
        const int ta = tile % tiles_a, tb = tile / tiles_a;
        const int kb0 = (int)((long long)kblocks * split / p.split_k);
        const int kb1 = (int)((long long)kblocks * (split + 1) / p.split_k);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kTimeoutEmptyBarrier, w);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = tiles + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          tma_load_2d_hint(sa, &tmap_a, &full_bar[stage], kb * kBK, ta * kBM, pol_a);
          tma_load_2d_hint(sb, &tmap_b, &full_bar[stage], kb * kBK, tb * BN, pol_b);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kBM, (uint32_t)p.umma_n, kFmtBF16, kFmtBF16);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int split = w % p.split_k;
        const int kb0 = (int)((long long)kblocks * split / p.split_k);
        const int kb1 = (int)((long long)kblocks * (split + 1) / p.split_k);
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1, abort_flag)) {
          report_status(p.status, kTimeoutTmemEmpty, w);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            report_status(p.status, kTimeoutFullBarrier, w);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * S::kStageBytes);
          const uint64_t da = make_desc_k_sw128(sa);
          const uint64_t db = make_desc_k_sw128(sa + S::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            umma_f16_ss(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);   // releases the smem stage when these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);       // accumulator complete
        acc_phase[acc] ^= 1;
        acc ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps (2..5)
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may access
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    for (int w = blockIdx.x; w < num_work; w += gridDim.x) {
      const int tile = w / p.split_k, split = w % p.split_k;
      const int ta = tile % tiles_a, tb = tile / tiles_a;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc], abort_flag)) {
        report_status(p.status, kTimeoutTmemFull, w);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      acc_phase[acc] ^= 1;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      const int i = ta * kBM + row_in_tile;
      const int j0 = tb * BN;
      const int ncols = min(BN, p.umma_n);
      constexpr int CH = (BN >= 32) ? 32 : 16;

      if (p.split_k == 1) {
#pragma unroll 1
        for (int c = 0; c < ncols; c += CH) {
          float v[CH];
          if constexpr (CH == 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = __uint_as_float(r[q]);
          } else {
            uint32_t r[16];
            tmem_ld_32x32b_x16(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(r[q]);
          }
          if (i < p.a_rows) {
            const float bias_i = (p.bias != nullptr && p.bias_on_a) ? __bfloat162float(p.bias[i]) : 0.f;
            __nv_bfloat16* orow = p.out + (long long)i * p.ldo_a;
            const int j = j0 + c;
            if (p.ldo_b == 1 && j + CH <= p.b_rows && ((reinterpret_cast<uintptr_t>(orow + j) & 15) == 0)) {
              uint32_t pk[CH / 2];
#pragma unroll
              for (int q = 0; q < CH; q += 2) {
                float b0 = bias_i, b1 = bias_i;
                if (p.bias != nullptr && !p.bias_on_a) {
                  b0 = __bfloat162float(p.bias[j + q]);
                  b1 = __bfloat162float(p.bias[j + q + 1]);
                }
                pk[q / 2] = pack_bf16x2(v[q] * p.out_scale + b0, v[q + 1] * p.out_scale + b1);
              }
              uint4* dst = reinterpret_cast<uint4*>(orow + j);
#pragma unroll
              for (int q = 0; q < CH / 8; ++q) dst[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            } else {
#pragma unroll
              for (int q = 0; q < CH; ++q) {
                if (j + q < p.b_rows) {
                  float b = bias_i;
                  if (p.bias != nullptr && !p.bias_on_a) b = __bfloat162float(p.bias[j + q]);
                  orow[(long long)(j + q) * p.ldo_b] = __float2bfloat16(v[q] * p.out_scale + b);
                }
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      } else {
        // ---- split-K: park the fp32 partial, count arrivals, the last CTA of the tile reduces.
        // Partial layout [split][column][128 rows]: for a fixed column the 32 lanes of a warp touch 32
        // consecutive floats, so both the parking stores and the reducer's loads are fully coalesced.
        float* __restrict__ wsp = p.ws + ((long long)(tile * p.split_k + split) * BN) * kBM + row_in_tile;
#pragma unroll 1
        for (int c = 0; c < ncols; c += CH) {
          if constexpr (CH == 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 32; ++q) __stcg(wsp + (long long)(c + q) * kBM, __uint_as_float(r[q]));
          } else {
            uint32_t r[16];
            tmem_ld_32x32b_x16(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 16; ++q) __stcg(wsp + (long long)(c + q) * kBM, __uint_as_float(r[q]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int prev = atomicAdd(&p.counters[tile], 1);
          *last_flag = (prev == p.split_k - 1) ? 1 : 0;
          if (prev == p.split_k - 1) p.counters[tile] = 0;   // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool is_last = (*last_flag != 0);
        if (is_last) {
          __threadfence();
          if (i < p.a_rows) {
            const float bias_i = (p.bias != nullptr && p.bias_on_a) ? __bfloat162float(p.bias[i]) : 0.f;
            __nv_bfloat16* __restrict__ orow = p.out + (long long)i * p.ldo_a;
            const float* __restrict__ base = p.ws + ((long long)(tile * p.split_k) * BN) * kBM + row_in_tile;
            const long long sstride = (long long)BN * kBM;
            constexpr int RC = 8;       // columns reduced together: RC * split independent loads in flight
#pragma unroll 1
            for (int c = 0; c < ncols; c += RC) {
              float acc8[RC];
#pragma unroll
              for (int q = 0; q < RC; ++q) acc8[q] = 0.f;
#pragma unroll 4
              for (int sp = 0; sp < p.split_k; ++sp) {
                float t[RC];
#pragma unroll
                for (int q = 0; q < RC; ++q) t[q] = __ldcg(base + sp * sstride + (long long)(c + q) * kBM);
#pragma unroll
                for (int q = 0; q < RC; ++q) acc8[q] += t[q];
              }
#pragma unroll
              for (int q = 0; q < RC; ++q) {
                const int j = j0 + c + q;
                if (j < p.b_rows) {
                  float b = bias_i;
                  if (p.bias != nullptr && !p.bias_on_a) b = __bfloat162float(p.bias[j]);
                  orow[(long long)j * p.ldo_b] = __float2bfloat16(acc8[q] * p.out_scale + b);
                }
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // last_flag is reused by the next tile
      }
      acc ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// 2-D K-major bf16 tensor map: dims {K, rows}, box {64, box_rows}, 128-byte swizzle, zero fill outside.
int make_tmap_bf16_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t K, uint64_t row_stride_elems,
                          uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int num_sms, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  const int tiles = ((p.a_rows + kBM - 1) / kBM) * ((p.b_rows + BN - 1) / BN);
  const int work = tiles * p.split_k;
  const int grid = work < num_sms ? work : num_sms;
  gemm_bf16_tcgen05_kernel<BN, STAGES><<<grid, kGemmThreads, S::kTotal, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// Pick the token tile (UMMA N) and the K split for the weights-on-M path with a small cost model.
// A work unit streams (128 + bn) * 2 * K / split bytes into shared memory (the weight tile from HBM, the token
// tile from L2); units run in waves of one per SM; a split adds the fp32 partial round trip plus the serial
// reduction by the last CTA.  Few tokens -> split K (partials are tiny); many tokens -> tile the tokens
// (partials would be large, while re-reading a weight tile from L2 is cheap).
static void choose_tile_and_split(int T, int N, int K, int num_sms, long long ws_bytes, int force_split, int force_bn, int* bn_out,
                                  int* split_out) {
  const int tiles_a = (N + kBM - 1) / kBM;
  const int kblocks = (K + kBK - 1) / kBK;
  int bn_full = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
  if (force_bn == 16 || force_bn == 32 || force_bn == 64 || force_bn == 128 || force_bn == 256) {
    if (force_bn < bn_full) bn_full = force_bn;
    if (force_split <= 0) force_split = 1;
  }
  if (force_split > 0) {            // tests and the no-allocation entry ask for an exact split on the full token tile
    int s = force_split > kblocks ? kblocks : force_split;
    const int tt = (T + bn_full - 1) / bn_full;
    if (s > 1 && ((long long)tiles_a * tt * s * kBM * bn_full * 4 > ws_bytes || tiles_a * tt > lx_gemm_max_tiles_const)) s = 1;
    *bn_out = bn_full;
    *split_out = s;
    return;
  }
  const int splits[] = {1, 2, 3, 4, 6, 8, 12, 16};
  double best = 1e30;
  int best_bn = bn_full, best_split = 1;
  for (int bn = bn_full; bn >= 16; bn >>= 1) {
    const int ttiles = (T + bn - 1) / bn;
    if (tiles_a * ttiles > lx_gemm_max_tiles_const) continue;
    for (int s : splits) {
      if (s > 1) {
        if (kblocks / s < 2) continue;
        if ((long long)tiles_a * ttiles * s * kBM * bn * 4 > ws_bytes) continue;
      }
      const long long units = (long long)tiles_a * ttiles * s;
      const double waves = (double)((units + num_sms - 1) / num_sms);
      const double fill = (double)(kBM + bn) * 2.0 * K / s;
      const double part = s > 1 ? (double)kBM * bn * 4.0 * 2.5 : 0.0;
      const double fixed = 48e3;
      const double tail = s > 1 ? (double)kBM * bn * 4.0 * s * 4.0 : 0.0;   // serial reduction by the last CTA (fitted to a sweep)
      const double cost = waves * (fill + part + fixed) + tail;
      if (cost < best) { best = cost; best_bn = bn; best_split = s; }
    }
  }
  *bn_out = best_bn;
  *split_out = best_split;
}

}  // namespace lx

extern "C" {

// Workspace sizes the caller must provide for split-K (bytes).
long long lx_gemm_ws_bytes() { return 64ll << 20; }
int lx_gemm_max_tiles() { return 8192; }

// out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N]).  `ldx`, `ldw`, `ldo` are row strides in elements.
// mode: 0 = choose, 1 = force weights on the M side (small T), 2 = force activations on the M side.
// Returns 0 or a negative error; device-side timeouts are reported through `status` (2 ints, zeroed by the caller).
int lx_gemm_bf16(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                 long long ldw, long long ldo, float out_scale, void* ws, long long ws_bytes, int* counters,
                 int* status, int num_sms, int mode, int force_split, void* stream_) {
  using namespace lx;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || N <= 0) return 0;
  if ((K % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return -1000;
  const bool swap = (mode == 1) || (mode == 0 && T <= 256);
  GemmParams p{};
  p.K = K;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.ws = reinterpret_cast<float*>(ws);
  p.counters = counters;
  p.status = status;
  p.out_scale = out_scale;
  p.split_k = 1;
  CUtensorMap ta, tb;
  int bn;
  if (swap) {
    if (T > 256) return -1001;
    p.a_rows = N; p.b_rows = T;
    p.ldo_a = 1; p.ldo_b = ldo;
    p.bias_on_a = 1;
    p.hint_a_first = 1;
    int split = 1;
    choose_tile_and_split(T, N, K, num_sms, (ws != nullptr && counters != nullptr) ? ws_bytes : 0, force_split & 0xffff, force_split >> 16, &bn, &split);
    p.umma_n = T >= bn ? bn : (T + 15) / 16 * 16;
    if (make_tmap_bf16_kmajor(&ta, w, N, K, ldw, kBM)) return -1002;
    if (make_tmap_bf16_kmajor(&tb, x, T, K, ldx, bn)) return -1003;
    p.split_k = split;
  } else {
    bn = 256;
    p.a_rows = T; p.b_rows = N;
    p.umma_n = 256;
    p.ldo_a = ldo; p.ldo_b = 1;
    p.bias_on_a = 0;
    p.hint_a_first = 0;
    if (make_tmap_bf16_kmajor(&ta, x, T, K, ldx, kBM)) return -1002;
    if (make_tmap_bf16_kmajor(&tb, w, N, K, ldw, bn)) return -1003;
  }
  switch (bn) {
    case 16:  return launch_gemm<16, 8>(ta, tb, p, num_sms, stream);
    case 32:  return launch_gemm<32, 8>(ta, tb, p, num_sms, stream);
    case 64:  return launch_gemm<64, 8>(ta, tb, p, num_sms, stream);
    case 128: return launch_gemm<128, 6>(ta, tb, p, num_sms, stream);
    default:  return launch_gemm<256, 4>(ta, tb, p, num_sms, stream);
  }
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in lx_noalloc.h).
//
// The split-K path above needs scratch: fp32 partial tiles plus one arrival counter per output tile.  The
// regular entry point takes that scratch from its caller.  Some callers cannot provide any: code that runs
// inside a stream capture, a real-time or safety-partitioned host that forbids cudaMalloc after start-up, a
// plugin living in another framework's process whose allocator it must not touch.  For them the same kernel is
// offered with its scratch in a fixed array that is part of this library's image.
//
// Limits, because the array is static: it is kNoAllocPartialBytes + kNoAllocCounters*4 + 16 bytes on EVERY
// GPU that loads this library, from load until the process exits.  Problems whose split-K partials would not
// fit are rejected (or, with split_k = 0, run with a smaller split that fits, down to no split at all).
// All calls share the one array and it keeps what the previous call left: the counters are cleared on the
// stream before every launch, the partials are fully overwritten before they are read.  Two calls that
// overlap on the GPU (different streams, or different host threads without ordering) would race on it.
// ------------------------------------------------------------------------------------------------
namespace lx {

constexpr long long kNoAllocPartialBytes = 8ll << 20;   // 8 MiB of fp32 partial tiles
constexpr int kNoAllocCounters = 1024;                  // one per 128-row output tile
constexpr int kNoAllocMaxDevices = 64;

struct NoAllocScratch {
  float partials[kNoAllocPartialBytes / 4];
  int counters[kNoAllocCounters];
  int status[4];
};

// In host code this name is only a handle for cudaGetSymbolAddress; it is NOT a device pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

// Device address of the array, per device, resolved on the first call made while that device is current.
static NoAllocScratch* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};

static int noalloc_scratch_for_current_device(NoAllocScratch** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return -2001;
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) return -2002;
    g_noalloc_ptr[dev] = reinterpret_cast<NoAllocScratch*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}

}  // namespace lx

extern "C" {

long long lx_gemm_bf16_noalloc_scratch_bytes() { return (long long)sizeof(lx::NoAllocScratch); }
int lx_gemm_bf16_noalloc_max_tokens() { return 256; }

const char* lx_gemm_bf16_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -2001: return "no current CUDA device (or device ordinal >= 64)";
    case -2002: return "cudaGetSymbolAddress failed for the static scratch array";
    case -2003: return "T exceeds the 256-token maximum of the no-allocation entry point";
    case -2004: return "N needs more than 1024 output tiles (N > 131072): beyond the static counter array";
    case -2005: return "requested split_k does not fit the 8 MiB static scratch for this N and T";
    case -2006: return "K, ldx and ldw must be multiples of 8 elements (16-byte TMA alignment)";
    case -2007: return "clearing the arrival counters failed";
    default: return "launch or tensor-map error (negative CUDA / driver code)";
  }
}

// out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N]), T <= 256, same math and the same kernel as lx_gemm_bf16 in its
// weights-on-M mode.  split_k: 0 = largest power of two that fits the static scratch and fills the GPU,
// otherwise the exact split to use (rejected with -2005 when its partials do not fit).
//
// The first call made on a device resolves the device address of the static array (cudaGetSymbolAddress) and
// sets the kernel's shared-memory attribute; make that first call outside any stream capture.  No cudaMalloc,
// cudaFree or other allocating routine is called, on any call.
int lx_gemm_bf16_noalloc(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                         long long ldw, long long ldo, int split_k, void* stream_) {
  using namespace lx;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || N <= 0) return 0;
  if (T > 256) return -2003;
  if ((K % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return -2006;
  NoAllocScratch* sc = nullptr;
  if (int rc = noalloc_scratch_for_current_device(&sc)) return rc;
  const int tiles = (N + kBM - 1) / kBM;
  if (tiles > kNoAllocCounters) return -2004;
  const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
  const int kblocks = (K + kBK - 1) / kBK;
  const long long per_split = (long long)tiles * kBM * bn * 4;
  int num_sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  if (num_sms <= 0) num_sms = 148;
  int split = 1;
  if (split_k > 0) {
    split = split_k > kblocks ? kblocks : split_k;
    if (split > 1 && per_split * split > kNoAllocPartialBytes) return -2005;
  } else {
    while (tiles * split < num_sms && kblocks / (split * 2) >= 4 && split < 16 && per_split * split * 2 <= kNoAllocPartialBytes) split *= 2;
  }
  GemmParams p{};
  p.K = K;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.ws = sc->partials;
  p.counters = sc->counters;
  p.status = sc->status;
  p.out_scale = 1.f;
  p.split_k = split;
  p.a_rows = N; p.b_rows = T;
  p.umma_n = (T + 15) / 16 * 16;
  p.ldo_a = 1; p.ldo_b = ldo;
  p.bias_on_a = 1;
  p.hint_a_first = 1;
  CUtensorMap ta, tb;
  if (make_tmap_bf16_kmajor(&ta, w, N, K, ldw, kBM)) return -1002;
  if (make_tmap_bf16_kmajor(&tb, x, T, K, ldx, bn)) return -1003;
  // The array keeps the previous call's contents: counters (and the status words) must start at zero.
  if (cudaMemsetAsync(sc->counters, 0, sizeof(int) * (kNoAllocCounters + 4), stream) != cudaSuccess) return -2007;
  switch (bn) {
    case 16:  return launch_gemm<16, 8>(ta, tb, p, num_sms, stream);
    case 32:  return launch_gemm<32, 8>(ta, tb, p, num_sms, stream);
    case 64:  return launch_gemm<64, 8>(ta, tb, p, num_sms, stream);
    case 128: return launch_gemm<128, 6>(ta, tb, p, num_sms, stream);
    default:  return launch_gemm<256, 4>(ta, tb, p, num_sms, stream);
  }
}

// Copies the two status words of the last launch on the current device to host memory (synchronises the device).
// 0 in out2[0] means every bounded wait inside the kernel completed.
int lx_gemm_bf16_noalloc_status(int* out2) {
  using namespace lx;
  NoAllocScratch* sc = nullptr;
  if (int rc = noalloc_scratch_for_current_device(&sc)) return rc;
  return -(int)cudaMemcpy(out2, sc->status, 2 * sizeof(int), cudaMemcpyDeviceToHost);
}

}  // extern "C"
