// Mixture-of-experts feed-forward on the device: routing, dispatch, grouped expert GEMMs, combine.
//
//   router logits   one warp per token: logits[t, e] = x[t, :] . Wr[e, :] in fp32
//   route + sort    softmax over all experts, top-k, renormalise the kept weights (the reference's routing math,
//                   server/lorax_server/models/custom_modeling/flash_mixtral_modeling.py:449-459), then the rows routed to each
//                   expert this rank owns become one contiguous run of a sorted order: seg[e] .. seg[e+1]
//   gather          xg[p, :] = x[token of sorted row p, :]
//   grouped GEMM    work items (expert, 128 features of its weight, token tile of its run) on tcgen05: weights on the UMMA M
//                   side through one tensor map over the experts' stacked matrices, tokens on N, accumulators in TMEM;
//                   a token tile that runs past its expert's rows computes a few columns nobody stores
//   combine         out[t, :] = sum_j w[t, j] * y[pos[t, j], :]
//
// Only the k experts a token was routed to do work for it (the reference gets that from megablocks' block-sparse kernels,
// flash_mixtral_modeling.py:517-666, and falls back to a dense all-experts bmm under 256 tokens, :668-722).  Every count lives
// on the device, every launch has static shapes (k * tokens rows at most), so a decode step with experts is one CUDA graph.
// Under expert parallelism a rank owns experts [e0, e0 + e_local): rows routed elsewhere get pos = -1 and the per-rank outputs
// are summed by the all-reduce that follows.
#include "common.cuh"

namespace lx {

constexpr int kMoeMaxExperts = 64;
constexpr int kMoeMaxK = 8;

// ------------------------------------------------------------------------------------------------ router logits
__global__ void __launch_bounds__(256) moe_router_logits_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                 const __nv_bfloat16* __restrict__ wr, long long ldw, float* __restrict__ logits,
                                                                 int T, int E, int H) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const __nv_bfloat16* xr = x + (long long)warp * ldx;
  for (int e = 0; e < E; ++e) {
    const __nv_bfloat16* w = wr + (long long)e * ldw;
    float acc = 0.f;
    for (int h = lane * 8; h < H; h += 32 * 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(xr + h);
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(w + h));
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fa = unpack_bf16x2(aw[q]), fb = unpack_bf16x2(bw[q]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) logits[(long long)warp * E + e] = acc;
  }
}

// ------------------------------------------------------------------------------------------------ route + sort
struct MoeRouteParams {
  const float* logits;     // [T, E]
  int T, E, k;
  int e0, e_local;
  int* topk_ids;           // [T, k]
  float* topk_w;           // [T, k]
  int* seg;                // [e_local + 1]
  int* pos;                // [T, k]
  int* sorted_tok;         // [T * k]
};

// One CTA does the whole step (T * E values): per-token top-k in registers, ranks inside an expert's run from shared-memory
// counters, a scan by one thread, then the final positions.  The order of rows inside a run depends on the order of the
// atomics; every row's result is independent of it and the combine sums a token's k contributions in index order.
__global__ void __launch_bounds__(1024) moe_route_kernel(const MoeRouteParams p) {
  pdl_wait();
  __shared__ int counts[kMoeMaxExperts];
  __shared__ int starts[kMoeMaxExperts + 1];
  if (threadIdx.x < kMoeMaxExperts) counts[threadIdx.x] = 0;
  __syncthreads();
  for (int t = threadIdx.x; t < p.T; t += blockDim.x) {
    const float* l = p.logits + (long long)t * p.E;
    float mx = -INFINITY;
    for (int e = 0; e < p.E; ++e) mx = fmaxf(mx, l[e]);
    float denom = 0.f;
    for (int e = 0; e < p.E; ++e) denom += __expf(l[e] - mx);
    int ids[kMoeMaxK];
    float pr[kMoeMaxK];
    float kept = 0.f;
    for (int j = 0; j < p.k; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < p.E; ++e) {
        bool taken = false;
        for (int q = 0; q < j; ++q) taken |= (ids[q] == e);
        const float v = l[e];
        if (!taken && v > bv) { bv = v; best = e; }       // ties go to the lower index, as torch.topk does on a sorted tie
      }
      ids[j] = best;
      pr[j] = __expf(bv - mx) / denom;
      kept += pr[j];
    }
    for (int j = 0; j < p.k; ++j) {
      p.topk_ids[t * p.k + j] = ids[j];
      p.topk_w[t * p.k + j] = pr[j] / kept;
      const int le = ids[j] - p.e0;
      p.pos[t * p.k + j] = (le >= 0 && le < p.e_local) ? atomicAdd(&counts[le], 1) : -1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < p.e_local; ++e) { starts[e] = run; run += counts[e]; }
    starts[p.e_local] = run;
    for (int e = 0; e <= p.e_local; ++e) p.seg[e] = starts[e];
  }
  __syncthreads();
  for (int t = threadIdx.x; t < p.T; t += blockDim.x) {
    for (int j = 0; j < p.k; ++j) {
      const int r = p.pos[t * p.k + j];
      if (r >= 0) {
        const int q = starts[p.topk_ids[t * p.k + j] - p.e0] + r;
        p.pos[t * p.k + j] = q;
        p.sorted_tok[q] = t;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ gather / combine
// xg[q, :] = x[sorted_tok[q], :] for the rows of the sorted order; one warp per row, 16 bytes per lane and pass.
__global__ void __launch_bounds__(256) moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ sorted_tok,
                                                         const int* __restrict__ seg, int e_local, __nv_bfloat16* __restrict__ xg, long long ldg,
                                                         int rows_cap, int H) {
  pdl_wait();
  const int total = min(seg[e_local], rows_cap);
  const int lane = threadIdx.x & 31;
  for (int q = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; q < total; q += (gridDim.x * blockDim.x) >> 5) {
    const __nv_bfloat16* src = x + (long long)sorted_tok[q] * ldx;
    __nv_bfloat16* dst = xg + (long long)q * ldg;
    for (int h = lane * 8; h < H; h += 256) *reinterpret_cast<uint4*>(dst + h) = *reinterpret_cast<const uint4*>(src + h);
  }
}

// out[t, :] = sum_j w[t, j] * y[pos[t, j], :] over the experts of the token that this rank owns (fp32 sum in index order).
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const int* __restrict__ pos,
                                                          const float* __restrict__ w, int k, __nv_bfloat16* __restrict__ out, long long ldo,
                                                          int T, int H) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += (gridDim.x * blockDim.x) >> 5) {
    for (int h = lane * 8; h < H; h += 256) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int j = 0; j < k; ++j) {
        const int q = pos[t * k + j];
        if (q < 0) continue;
        const float wj = w[t * k + j];
        const uint4 v = *reinterpret_cast<const uint4*>(y + (long long)q * ldy + h);
        const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 f = unpack_bf16x2(vw[u]);
          acc[2 * u] = fmaf(wj, f.x, acc[2 * u]);
          acc[2 * u + 1] = fmaf(wj, f.y, acc[2 * u + 1]);
        }
      }
      *reinterpret_cast<uint4*>(out + (long long)t * ldo + h) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
}

// ------------------------------------------------------------------------------------------------ grouped GEMM
constexpr int kMgBM = 128;
constexpr int kMgBK = 64;
constexpr int kMgThreads = 192;

struct MoeGemmParams {
  int K, n_w, e_local;
  const int* seg;                 // [e_local + 1] rows of every local expert in the sorted order
  __nv_bfloat16* out;             // [rows, n_w]
  long long ldo;
  int bn;                         // token tile = UMMA N (multiple of 16, <= BN)
  int rows_cap;                   // rows the buffers hold
  int* status;
};

template <int BN, int STAGES>
struct MgSmem {
  static constexpr int kABytes = kMgBM * kMgBK * 2;
  static constexpr int kBBytes = BN * kMgBK * 2;
  static constexpr int kStage = kABytes + kBBytes;
  static constexpr int kTotal = STAGES * kStage + 1024 + 1024;
};

// Work item g -> (expert, feature tile, token tile).  Token tiles of one (expert, feature tile) are adjacent, so CTAs that run
// side by side read the same weight tile through L2 and it leaves HBM once.
struct MgIter {
  int e_local, tiles_a, bn;
  int cum[kMoeMaxExperts + 1];    // tiles before expert e
  int start[kMoeMaxExperts + 1];
  __device__ void init(const MoeGemmParams& p, const int* seg_s) {
    e_local = p.e_local; tiles_a = p.n_w / kMgBM; bn = p.bn;
    int run = 0;
    for (int e = 0; e < e_local; ++e) {
      start[e] = seg_s[e];
      cum[e] = run;
      const int cnt = min(seg_s[e + 1], p.rows_cap) - min(seg_s[e], p.rows_cap);
      run += tiles_a * ((cnt + bn - 1) / bn);
    }
    start[e_local] = min(seg_s[e_local], p.rows_cap);
    cum[e_local] = run;
  }
  __device__ int total() const { return cum[e_local]; }
  __device__ void decode(int g, int& e, int& ta, int& tb, int& row0, int& nrows) const {
    e = 0;
    while (e + 1 < e_local && g >= cum[e + 1]) ++e;
    const int local = g - cum[e];
    const int cnt = start[e + 1] - start[e];
    const int nt = (cnt + bn - 1) / bn;
    ta = local / nt;
    tb = local - ta * nt;
    row0 = start[e] + tb * bn;
    nrows = min(bn, cnt - tb * bn);
  }
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kMgThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const MoeGemmParams p) {
  using S = MgSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStage);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* seg_s = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 4));       // [e_local + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  const int kblocks = (p.K + kMgBK - 1) / kMgBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tmem_full[s], 1); mbar_init(&tmem_empty[s], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  if ((int)threadIdx.x <= p.e_local) seg_s[threadIdx.x] = p.seg[threadIdx.x];
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      MgIter it;
      it.init(p, seg_s);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int g = (int)blockIdx.x; ok && g < it.total(); g += (int)gridDim.x) {
        int e, ta, tb, row0, nrows;
        it.decode(g, e, ta, tb, row0, nrows);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { report_status(p.status, kTimeoutEmptyBarrier, g); *abort_flag = 1; ok = false; break; }
          uint8_t* sa = tiles + stage * S::kStage;
          mbar_expect_tx(&full_bar[stage], (uint32_t)(S::kABytes + p.bn * kMgBK * 2));
          tma_load_2d_hint(sa, &tmap_w, &full_bar[stage], kb * kMgBK, e * p.n_w + ta * kMgBM, pol_w);
          tma_load_2d_hint(sa + S::kABytes, &tmap_x, &full_bar[stage], kb * kMgBK, row0, pol_x);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kMgBM, (uint32_t)p.bn, kFmtBF16, kFmtBF16);
      MgIter it;
      it.init(p, seg_s);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase[2] = {0, 0};
      bool ok = true;
      for (int g = (int)blockIdx.x; ok && g < it.total(); g += (int)gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1, abort_flag)) { report_status(p.status, kTimeoutTmemEmpty, g); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { report_status(p.status, kTimeoutFullBarrier, g); *abort_flag = 1; ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * S::kStage);
          const uint64_t da = make_desc_k_sw128(sa), db = make_desc_k_sw128(sa + S::kABytes);
#pragma unroll
          for (int k = 0; k < kMgBK / 16; ++k) umma_f16_ss(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);
        acc_phase[acc] ^= 1;
        acc ^= 1;
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    MgIter it;
    it.init(p, seg_s);
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    for (int g = (int)blockIdx.x; g < it.total(); g += (int)gridDim.x) {
      int e, ta, tb, row0, nrows;
      it.decode(g, e, ta, tb, row0, nrows);
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc], abort_flag)) { report_status(p.status, kTimeoutTmemFull, g); *abort_flag = 1; break; }
      tc_fence_after();
      acc_phase[acc] ^= 1;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      const int i = ta * kMgBM + quad * 32 + lane;             // feature of this lane
      constexpr int CH = (BN >= 32) ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < p.bn; c += CH) {
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
        if (i < p.n_w) {
#pragma unroll
          for (int q = 0; q < CH; ++q) {
            if (c + q < nrows) p.out[(long long)(row0 + c + q) * p.ldo + i] = __float2bfloat16(v[q]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

int make_tmap_bf16_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t K, uint64_t row_stride_elems, uint32_t box_rows);

template <int BN, int STAGES>
static int launch_moe_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const MoeGemmParams& p, int grid, cudaStream_t stream) {
  using S = MgSmem<BN, STAGES>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -(int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  launch_pdl(moe_grouped_gemm_kernel<BN, STAGES>, dim3(grid), dim3(kMgThreads), (size_t)S::kTotal, stream, tw, tx, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace lx

extern "C" {

// logits[T, E] (fp32) = x[T, H] @ wr[E, H]^T
int lx_moe_router_logits(const void* x, long long ldx, const void* wr, long long ldw, float* logits, int T, int E, int H, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return -1;
  launch_pdl(moe_router_logits_kernel, dim3((T * 32 + 255) / 256), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
             reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(wr), ldw, logits, T, E, H);
  return -(int)cudaGetLastError();
}

// Softmax -> top-k -> renormalise -> sorted order of the rows routed to experts [e0, e0 + e_local).
int lx_moe_route(const float* logits, int T, int E, int k, int e0, int e_local, int* topk_ids, float* topk_w, int* seg, int* pos,
                 int* sorted_tok, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (E > kMoeMaxExperts || k > kMoeMaxK || k > E || e_local > kMoeMaxExperts) return -1;
  MoeRouteParams p{logits, T, E, k, e0, e_local, topk_ids, topk_w, seg, pos, sorted_tok};
  launch_pdl(moe_route_kernel, dim3(1), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), p);
  return -(int)cudaGetLastError();
}

int lx_moe_gather(const void* x, long long ldx, const int* sorted_tok, const int* seg, int e_local, void* xg, long long ldg, int rows_cap, int H,
                  void* stream) {
  using namespace lx;
  if (rows_cap <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldg % 8 != 0) return -1;
  const int blocks = min((rows_cap * 32 + 255) / 256, 148 * 8);
  launch_pdl(moe_gather_kernel, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(x), ldx,
             sorted_tok, seg, e_local, reinterpret_cast<__nv_bfloat16*>(xg), ldg, rows_cap, H);
  return -(int)cudaGetLastError();
}

int lx_moe_combine(const void* y, long long ldy, const int* pos, const float* w, int k, void* out, long long ldo, int T, int H, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldy % 8 != 0 || ldo % 8 != 0) return -1;
  const int blocks = min((T * 32 + 255) / 256, 148 * 8);
  launch_pdl(moe_combine_kernel, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(y), ldy,
             pos, w, k, reinterpret_cast<__nv_bfloat16*>(out), ldo, T, H);
  return -(int)cudaGetLastError();
}

// out[q, :] = xg[q, :] @ W_e(q)^T for every sorted row q, e(q) the expert whose run holds q.  w: the experts' matrices stacked
// [e_local * n_w, K]; n_w must be a multiple of 128.  avg_rows (rows per expert the caller expects) picks the token tile.
int lx_moe_grouped_gemm(const void* xg, long long ldx, const void* w, long long ldw, void* out, long long ldo, const int* seg, int e_local,
                        int rows_cap, int n_w, int K, int avg_rows, int* status, int num_sms, void* stream) {
  using namespace lx;
  if (rows_cap <= 0 || e_local <= 0) return 0;
  if (n_w % kMgBM != 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || e_local > kMoeMaxExperts) return -1;
  int bn = (avg_rows + 15) / 16 * 16;
  if (bn < 16) bn = 16;
  if (bn > 256) bn = 256;
  const int tbn = bn <= 16 ? 16 : bn <= 32 ? 32 : bn <= 64 ? 64 : bn <= 128 ? 128 : 256;
  MoeGemmParams p{};
  p.K = K; p.n_w = n_w; p.e_local = e_local; p.seg = seg;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.bn = bn; p.rows_cap = rows_cap; p.status = status;
  CUtensorMap tw, tx;
  if (make_tmap_bf16_kmajor(&tw, w, (uint64_t)e_local * n_w, K, ldw, kMgBM)) return -2;
  if (make_tmap_bf16_kmajor(&tx, xg, rows_cap, K, ldx, bn)) return -3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (tbn) {
    case 16:  return launch_moe_gemm<16, 8>(tw, tx, p, num_sms, s);
    case 32:  return launch_moe_gemm<32, 8>(tw, tx, p, num_sms, s);
    case 64:  return launch_moe_gemm<64, 8>(tw, tx, p, num_sms, s);
    case 128: return launch_moe_gemm<128, 6>(tw, tx, p, num_sms, s);
    default:  return launch_moe_gemm<256, 4>(tw, tx, p, num_sms, s);
  }
}

}  // extern "C"
