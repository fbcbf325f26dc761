// Segmented multi-adapter LoRA on the tensor cores.
//
// Tokens of a step are ordered so that tokens of the same adapter are adjacent (the runtime keeps decode rows
// sorted by adapter slot; in prefill a request's tokens are adjacent anyway).  The host describes the step as a
// table of tiles  {slot, first row, rows (<= BN), -}  and every tile is one CTA:
//
//   shrink   D[R, n] = A_cat(slot)[R, K] * X[row0 .. row0+n, K]^T        tcgen05.mma, M = 128 (R rows live,
//            the rest zero-filled by TMA), N = tokens of the tile, accumulator in TMEM, both operands by TMA:
//            the adapter matrix through a per-slot 3-D tensor map {K, R, layer} that the adapter manager encodes
//            when the adapter becomes resident, the activations through a per-launch 2-D map.
//   expand   y[row, n] += sum_j v[row, part(n) * r + j] * B_cat(slot)[n, j]   K = r is tiny (8..64): a SIMT kernel
//            that keeps a B row pair in registers and walks the tile's tokens, coalesced read-modify-write of y.
//
// One launch of each serves any mix of adapters and ranks.  They replace the reference's SGMV shrink / CUTLASS
// grouped-GEMM expand pair that is launched once per distinct rank (server/punica_kernels/punica_kernels/
// sgmv_flashinfer/sgmv_flashinfer.cuh:13-353, sgmv/sgmv_cutlass.cuh:31-179, utils/layers.py:114-164).
#include "common.cuh"

namespace lx {

constexpr int kLtThreads = 192;
constexpr int kLtBK = 64;

struct LoraTile { int slot, row0, nrows, pad; };

LX_DEVICE void tensormap_fence_acquire(const CUtensorMap* m) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

struct ShrinkTcParams {
  const LoraTile* tiles;
  const CUtensorMap* slot_tmaps;   // [num_slots][groups_per_slot]
  int groups_per_slot, group;
  const int* slot_rank;
  int num_slots;
  int nparts;                      // R = nparts * rank
  int layer;
  float* v;                        // [ksplit][v_rows][ldv] fp32 partial sums of the K splits (unused when ksplit == 1)
  int ldv;
  long long v_split_stride;        // elements between two K-splits
  int ksplit;
  float* v_final;                  // [v_rows][ldv] the result: the last split CTA of a tile sums the partials in split order
  int* counters;                   // one arrival counter per (tile, row chunk), zero between launches
  int K, T;
  int* status;
};

// Shared-memory plan.  The adapter tile of a stage only occupies box_rows * 128 bytes (box_rows = R rounded up to
// 16), so the stage stride is chosen at run time from the slot's rank and the ring gets as many stages as fit:
// small ranks get a deep ring, which is what hides the TMA latency of these skinny tiles.  The MMA always reads
// 128 rows (16 KB) from the stage base; the rows past box_rows belong to later stages (or to the 16 KB of slack
// after the ring) and only feed accumulator rows that are never stored.
constexpr int kLtMaxStages = 12;
template <int BN>
struct LtSmem {
  static constexpr int kBBytes = BN * kLtBK * 2;
  static constexpr int kRing = BN <= 32 ? 80 * 1024 : 176 * 1024;
  static constexpr int kSlack = 16 * 1024;
  static constexpr int kTotal = kRing + kSlack + 512 + 1024;
};

template <int BN>
__global__ void __launch_bounds__(kLtThreads)
lora_shrink_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const ShrinkTcParams p) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  using S = LtSmem<BN>;
  LoraTile tile = p.tiles[blockIdx.x];
  tile.nrows = min(tile.nrows, p.T - tile.row0);       // a table may be older than the batch: rows past T are gone
  if (tile.slot < 0 || tile.nrows <= 0) return;
  if (tile.slot >= p.num_slots) {
    if (threadIdx.x == 0) report_status(p.status, kBadIndex, tile.slot);
    return;
  }
  const int r = p.slot_rank[tile.slot];
  const int R = r * p.nparts;
  const int m0 = blockIdx.y * 128;           // rows of A_cat handled by this CTA
  if (m0 >= R) return;
  const int box_rows = min(128, (R + 15) / 16 * 16);   // must match the encoder (lx_lora_encode_tmap)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = (box_rows * kLtBK * 2 + 1023) & ~1023;
  const int stage_stride = a_bytes + S::kBBytes;
  const int STAGES = min(kLtMaxStages, S::kRing / stage_stride);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kRing + S::kSlack);
  uint64_t* empty_bar = full_bar + kLtMaxStages;
  uint64_t* done_bar = empty_bar + kLtMaxStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kCols = BN < 32 ? 32 : BN;
  const CUtensorMap* tmap_a = p.slot_tmaps + (long long)tile.slot * p.groups_per_slot + p.group;
  const int kblocks_all = (p.K + kLtBK - 1) / kLtBK;
  const int kb_begin = (int)((long long)kblocks_all * blockIdx.z / p.ksplit);
  const int kb_end = (int)((long long)kblocks_all * (blockIdx.z + 1) / p.ksplit);
  const int kblocks = kb_end - kb_begin;
  float* __restrict__ vout = p.ksplit > 1 ? p.v + (long long)blockIdx.z * p.v_split_stride : p.v_final;
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tensormap_fence_acquire(tmap_a);
      const uint64_t pol_a = policy_evict_first(), pol_x = policy_evict_last();
      const uint32_t bytes = (uint32_t)(box_rows * kLtBK * 2 + S::kBBytes);
      int stage = 0; uint32_t phase = 0;
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { report_status(p.status, kTimeoutEmptyBarrier, blockIdx.x); *abort_flag = 1; break; }
        uint8_t* sa = smem + stage * stage_stride;
        mbar_expect_tx(&full_bar[stage], bytes);
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
            ::"r"(smem_u32(sa)), "l"(reinterpret_cast<uint64_t>(tmap_a)), "r"(smem_u32(&full_bar[stage])), "r"((kb_begin + kb) * kLtBK), "r"(m0),
              "r"(p.layer), "l"(pol_a) : "memory");
        tma_load_2d_hint(sa + a_bytes, &tmap_x, &full_bar[stage], (kb_begin + kb) * kLtBK, tile.row0, pol_x);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(128, (uint32_t)BN, kFmtBF16, kFmtBF16);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { report_status(p.status, kTimeoutFullBarrier, blockIdx.x); *abort_flag = 1; ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * stage_stride);
        const uint64_t da = make_desc_k_sw128(sa), db = make_desc_k_sw128(sa + a_bytes);
#pragma unroll
        for (int k = 0; k < kLtBK / 16; ++k) umma_f16_ss(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(&empty_bar[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) tc_commit(done_bar);
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int j = m0 + quad * 32 + lane;           // row of A_cat = column of v
    if (mbar_wait(done_bar, 0, abort_flag)) {
      tc_fence_after();
      const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16);
      constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < BN && c < tile.nrows; c += CH) {
        float vals[CH];
        if constexpr (CH == 32) {
          uint32_t rr[32];
          tmem_ld_32x32b_x32(taddr + c, rr);
          tc_wait_ld();
#pragma unroll
          for (int q = 0; q < 32; ++q) vals[q] = __uint_as_float(rr[q]);
        } else {
          uint32_t rr[16];
          tmem_ld_32x32b_x16(taddr + c, rr);
          tc_wait_ld();
#pragma unroll
          for (int q = 0; q < 16; ++q) vals[q] = __uint_as_float(rr[q]);
        }
        if (j < R) {
#pragma unroll
          for (int q = 0; q < CH; ++q) {
            if (c + q < tile.nrows) vout[(long long)(tile.row0 + c + q) * p.ldv + j] = vals[q];
          }
        }
      }
      if (p.ksplit > 1) {
        // The K splits of a tile finish in any order; whichever arrives last adds them up in split order, so the
        // result does not depend on the order of arrival.
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          int* ctr = p.counters + blockIdx.x * gridDim.y + blockIdx.y;
          const int prev = atomicAdd(ctr, 1);
          *last_flag = (prev == p.ksplit - 1) ? 1 : 0;
          if (prev == p.ksplit - 1) *ctr = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag != 0 && j < R) {
          __threadfence();
          constexpr int QU = 8;           // rows summed together: QU * ksplit independent loads in flight
          for (int q0 = 0; q0 < tile.nrows; q0 += QU) {
            float acc[QU];
#pragma unroll
            for (int u = 0; u < QU; ++u) acc[u] = 0.f;
            for (int sp = 0; sp < p.ksplit; ++sp) {
              float t[QU];
#pragma unroll
              for (int u = 0; u < QU; ++u) {
                const int q = min(q0 + u, tile.nrows - 1);
                t[u] = __ldcg(p.v + (long long)sp * p.v_split_stride + (long long)(tile.row0 + q) * p.ldv + j);
              }
#pragma unroll
              for (int u = 0; u < QU; ++u) acc[u] += t[u];
            }
#pragma unroll
            for (int u = 0; u < QU; ++u) {
              if (q0 + u < tile.nrows) p.v_final[(long long)(tile.row0 + q0 + u) * p.ldv + j] = acc[u];
            }
          }
        }
      }
    } else {
      report_status(p.status, kTimeoutTmemFull, blockIdx.x);
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_d, kCols); }
}

// ------------------------------------------------------------------------------------------------ expand
struct ExpandTiledParams {
  const LoraTile* tiles;
  const __nv_bfloat16* arena;
  const long long* slot_base;
  const int* slot_rank;
  int num_slots;
  long long unit_off;
  const float* v;                  // [T, ldv] shrink result
  int ldv;
  __nv_bfloat16* y;
  long long ldy;
  int n0, n1, N, T;
  int num_tiles, col_blocks;
  int* status;
};

constexpr int kExpThreads = 256;
constexpr int kExpCols = 4;                          // adjacent output features per thread: 128 contiguous bytes of B_cat at rank 16
constexpr int kExpBlockCols = kExpThreads * kExpCols;
constexpr int kExpMaxRows = 128;                     // rows of a tile staged at once
constexpr int kExpStage = 16;                        // ranks per pass
constexpr int kExpRowsInFlight = 4;                  // rows whose y loads are issued together

// One unit of work = one tile (a run of rows of one adapter) x 1024 output features.  A thread keeps the B_cat rows
// of its four features in registers (16 ranks at a time, packed bf16) and walks the rows of the tile: v comes from
// shared memory as broadcasts, y is read and written 8 bytes per thread, 256 contiguous bytes per warp.  The loads
// of B, of v and of the first rows of y are all issued before the first barrier, so a unit costs about one trip to
// memory.  Ranks above 16 take one pass over the tile's rows per 16 ranks.
//
// The grid is a fixed number of CTAs that walk the units; live tiles come first in the table, so the walk stops at
// the first dead one and padding entries cost nothing.
__global__ void __launch_bounds__(kExpThreads, 2) lora_expand_tiled_kernel(const ExpandTiledParams p) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  __shared__ __align__(16) float vs[kExpMaxRows * 3 * kExpStage];   // [row][part][16]
  const int nparts = p.n1 < p.N ? 3 : (p.n0 < p.N ? 2 : 1);
  for (int w = blockIdx.x; w < p.num_tiles * p.col_blocks; w += gridDim.x) {
    const LoraTile tile = p.tiles[w / p.col_blocks];
    if (tile.slot < 0) break;
    if (tile.nrows <= 0) continue;
    if (tile.slot >= p.num_slots) {
      if (threadIdx.x == 0) report_status(p.status, kBadIndex, tile.slot);
      continue;
    }
    const int r = p.slot_rank[tile.slot];
    const long long base = p.slot_base[tile.slot];
    if (base < 0 || r <= 0) continue;
    const int n = (w % p.col_blocks) * kExpBlockCols + threadIdx.x * kExpCols;
    const bool col_ok = n < p.N;                        // N is a multiple of 4: a thread's four features are all in or all out
    const int part = n < p.n0 ? 0 : (n < p.n1 ? 1 : 2);
    const __nv_bfloat16* B = p.arena + base + (long long)r * p.unit_off + (long long)n * r;
    const int nrows = min(min(tile.nrows, kExpMaxRows), p.T - tile.row0);
    if (nrows <= 0) continue;
    __nv_bfloat16* yrow0 = p.y + (long long)tile.row0 * p.ldy + n;

    for (int jc = 0; jc < r; jc += kExpStage) {
      const int rs = min(kExpStage, r - jc);            // 8 or 16 live ranks in this pass
      uint4 bw[kExpCols][kExpStage / 8];
#pragma unroll
      for (int c = 0; c < kExpCols; ++c) {
#pragma unroll
        for (int h = 0; h < kExpStage / 8; ++h) {
          bw[c][h] = make_uint4(0u, 0u, 0u, 0u);
          if (col_ok && h * 8 < rs) bw[c][h] = __ldg(reinterpret_cast<const uint4*>(B + (long long)c * r + jc + h * 8));
        }
      }
      uint2 old[kExpRowsInFlight];
#pragma unroll
      for (int u = 0; u < kExpRowsInFlight; ++u) {
        if (col_ok && u < nrows) old[u] = *reinterpret_cast<const uint2*>(yrow0 + (long long)u * p.ldy);
      }
      // stage v[row][part][jc .. jc+16) (zeros past the rank)
      __syncthreads();                                   // the previous unit's readers are done with vs
      for (int e = threadIdx.x; e < nrows * nparts * kExpStage; e += kExpThreads) {
        const int j = e % kExpStage, pr = e / kExpStage;
        const int pp = pr % nparts, m = pr / nparts;
        vs[(m * 3 + pp) * kExpStage + j] = (j < rs) ? p.v[(long long)(tile.row0 + m) * p.ldv + pp * r + jc + j] : 0.f;
      }
      __syncthreads();
      if (col_ok) {
        for (int m0 = 0; m0 < nrows; m0 += kExpRowsInFlight) {
          uint2 nxt[kExpRowsInFlight];
#pragma unroll
          for (int u = 0; u < kExpRowsInFlight; ++u) {      // next group's y while this one is computed
            const int m = m0 + kExpRowsInFlight + u;
            if (m < nrows) nxt[u] = *reinterpret_cast<const uint2*>(yrow0 + (long long)m * p.ldy);
          }
#pragma unroll
          for (int u = 0; u < kExpRowsInFlight; ++u) {
            if (m0 + u < nrows) {
              const float4* vp = reinterpret_cast<const float4*>(vs + ((m0 + u) * 3 + part) * kExpStage);
              float acc[kExpCols] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
              for (int h = 0; h < kExpStage / 8; ++h) {
                const float4 va = vp[2 * h], vb = vp[2 * h + 1];
#pragma unroll
                for (int c = 0; c < kExpCols; ++c) {
                  const float2 b0 = unpack_bf16x2(bw[c][h].x), b1 = unpack_bf16x2(bw[c][h].y);
                  const float2 b2 = unpack_bf16x2(bw[c][h].z), b3 = unpack_bf16x2(bw[c][h].w);
                  acc[c] = fmaf(va.x, b0.x, acc[c]); acc[c] = fmaf(va.y, b0.y, acc[c]);
                  acc[c] = fmaf(va.z, b1.x, acc[c]); acc[c] = fmaf(va.w, b1.y, acc[c]);
                  acc[c] = fmaf(vb.x, b2.x, acc[c]); acc[c] = fmaf(vb.y, b2.y, acc[c]);
                  acc[c] = fmaf(vb.z, b3.x, acc[c]); acc[c] = fmaf(vb.w, b3.y, acc[c]);
                }
              }
              const float2 o0 = unpack_bf16x2(old[u].x), o1 = unpack_bf16x2(old[u].y);
              uint2 nw;
              nw.x = pack_bf16x2(o0.x + acc[0], o0.y + acc[1]);
              nw.y = pack_bf16x2(o1.x + acc[2], o1.y + acc[3]);
              *reinterpret_cast<uint2*>(yrow0 + (long long)(m0 + u) * p.ldy) = nw;
            }
          }
#pragma unroll
          for (int u = 0; u < kExpRowsInFlight; ++u) old[u] = nxt[u];
        }
      }
    }
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn2 encode_fn2() {
  static EncodeTiledFn2 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn2>(ptr);
  }
  return fn;
}

template <int BN>
static int launch_shrink_tc(const CUtensorMap& tx, const ShrinkTcParams& p, int num_tiles, int chunks, cudaStream_t s) {
  using S = LtSmem<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(lora_shrink_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  dim3 grid(num_tiles, chunks, p.ksplit);
  launch_pdl(lora_shrink_tc_kernel<BN>, grid, dim3(kLtThreads), (size_t)S::kTotal, s, tx, p);
  return -(int)cudaGetLastError();
}

}  // namespace lx

extern "C" {

int lx_tensormap_bytes() { return (int)sizeof(CUtensorMap); }

// Encode the tensor map of one adapter matrix family: A_cat of every layer of one projection group.
//   base: device address of layer 0's A_cat [R, K]; layer l is `layer_stride` elements further.
// The 128-byte result is written to host memory at `out`; the caller copies it into the device table.
int lx_lora_encode_tmap(void* out, const void* base, int K, int R, long long layer_stride, int layers) {
  using namespace lx;
  EncodeTiledFn2 fn = encode_fn2();
  if (fn == nullptr) return -1;
  if ((K % 8) != 0 || (layer_stride % 8) != 0 || (reinterpret_cast<uintptr_t>(base) & 15)) return -2;
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)R, (cuuint64_t)layers};
  cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)layer_stride * 2};
  const cuuint32_t box_rows = (cuuint32_t)((R + 15) / 16 * 16 < 128 ? (R + 15) / 16 * 16 : 128);
  cuuint32_t box[3] = {(cuuint32_t)kLtBK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

// Tensor map of one B_cat family for the GEMM that adds the LoRA delta by UMMAs: {r, N, layers} read in boxes of 16 ranks x
// 128 features with the 32-byte swizzle (one K slice of a UMMA operand).  base: layer 0's B_cat [N, r].
int lx_lora_encode_tmap_b(void* out, const void* base, int r, int N, long long layer_stride, int layers) {
  using namespace lx;
  EncodeTiledFn2 fn = encode_fn2();
  if (fn == nullptr) return -1;
  if ((r % 8) != 0 || (layer_stride % 8) != 0 || (reinterpret_cast<uintptr_t>(base) & 15)) return -2;
  cuuint64_t dims[3] = {(cuuint64_t)r, (cuuint64_t)N, (cuuint64_t)layers};
  cuuint64_t strides[2] = {(cuuint64_t)r * 2, (cuuint64_t)layer_stride * 2};
  cuuint32_t box[3] = {16, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -(int)rc - 100;
}

// v[T, ldv] = x[T, K] @ A_cat(slot)^T for every tile of the table.  max_tile_rows selects the token-tile width
// (<= 32: decode, <= 128: prefill); max_rank bounds the number of 128-row chunks of A_cat.
int lx_lora_shrink_tc(const void* x, long long ldx, const void* tiles, int num_tiles, int max_tile_rows, const void* slot_tmaps,
                      int groups_per_slot, int group, const int* slot_rank, int num_slots, int nparts, int layer, float* v, int ldv,
                      long long v_split_stride, int ksplit, float* v_final, int* counters, int num_counters, int T, int K, int max_rank,
                      int* status, void* stream) {
  using namespace lx;
  if (num_tiles <= 0 || max_rank <= 0) return 0;
  if (K % 8 != 0 || ldx % 8 != 0 || nparts * max_rank > ldv) return -1;
  ShrinkTcParams p{};
  p.tiles = reinterpret_cast<const LoraTile*>(tiles);
  p.slot_tmaps = reinterpret_cast<const CUtensorMap*>(slot_tmaps);
  p.groups_per_slot = groups_per_slot; p.group = group; p.slot_rank = slot_rank; p.num_slots = num_slots;
  p.nparts = nparts; p.layer = layer; p.v = v; p.ldv = ldv; p.K = K; p.T = T; p.status = status;
  p.v_split_stride = v_split_stride;
  p.ksplit = ksplit < 1 ? 1 : ksplit;
  if (p.ksplit > (K + kLtBK - 1) / kLtBK) p.ksplit = (K + kLtBK - 1) / kLtBK;
  const int chunks = (nparts * max_rank + 127) / 128;
  if (counters == nullptr || num_tiles * chunks > num_counters || v == nullptr) p.ksplit = 1;
  p.v_final = v_final; p.counters = counters;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int bn = max_tile_rows <= 32 ? 32 : 128;
  // activations: 2-D K-major map with a BN-row box (same encoding as the GEMM's operands)
  EncodeTiledFn2 fn = encode_fn2();
  if (fn == nullptr) return -2;
  CUtensorMap tx;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)T};
  cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
  cuuint32_t box[2] = {(cuuint32_t)kLtBK, (cuuint32_t)bn};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -3;
  if (bn == 32) return launch_shrink_tc<32>(tx, p, num_tiles, chunks, s);
  return launch_shrink_tc<128>(tx, p, num_tiles, chunks, s);
}

int lx_lora_expand_tiled(const float* v, int ldv, long long v_split_stride, int ksplit, const void* tiles, int num_tiles,
                         int max_tile_rows, const void* arena, const long long* slot_base, const int* slot_rank, int num_slots,
                         long long unit_off, void* y, long long ldy, int T, int N, int n0, int n1, int* status, void* stream) {
  using namespace lx;
  (void)v_split_stride;
  if (num_tiles <= 0) return 0;
  if ((N | n0 | n1) & 3 || ldy % 4 != 0 || (reinterpret_cast<uintptr_t>(y) & 7) != 0) return -1;
  if (ksplit != 1 || max_tile_rows > kExpMaxRows) return -2;          // the shrink hands over the summed result
  ExpandTiledParams p{};
  p.tiles = reinterpret_cast<const LoraTile*>(tiles);
  p.arena = reinterpret_cast<const __nv_bfloat16*>(arena);
  p.slot_base = slot_base; p.slot_rank = slot_rank; p.num_slots = num_slots; p.unit_off = unit_off;
  p.v = v; p.ldv = ldv; p.y = reinterpret_cast<__nv_bfloat16*>(y); p.ldy = ldy; p.n0 = n0; p.n1 = n1; p.N = N; p.T = T;
  p.status = status;
  p.num_tiles = num_tiles;
  p.col_blocks = (N + kExpBlockCols - 1) / kExpBlockCols;
  const long long work = (long long)num_tiles * p.col_blocks;
  const int grid = (int)(work < 148 * 2 ? work : 148 * 2);
  launch_pdl(lora_expand_tiled_kernel, dim3(grid), dim3(kExpThreads), 0, reinterpret_cast<cudaStream_t>(stream), p);
  return -(int)cudaGetLastError();
}

}  // extern "C"
