// Two-shot all-reduce over NVLink peer memory for tensor-parallel activations (bf16 [tokens, hidden]).
//
// Every rank owns one symmetric buffer (same layout on every GPU, mapped into every process): an input area that the
// row-parallel GEMM writes its partial result into, an output area, and barrier flags.  One launch per rank:
//
//   A  each block announces "my input is written" to the same block of every rank (one release store per rank, issued by
//      different threads) and waits for all of them;
//   B  the rank reduces ITS slice (1 / world of the elements): 16-byte loads of that slice from every rank's input
//      over NVLink, fp32 sum in rank order (so every element has one owner and the result is bit-identical everywhere),
//      16-byte stores of the bf16 result into every rank's output area;
//   C  each block announces "my stores are done" and waits for its counterparts, so that when the kernel completes
//      the whole output area of this rank has been written by its owners and nobody still reads this rank's input.
//
// This replaces `dist.all_reduce` (NCCL) after the O and down projections (call sites C2 / C3 / C5 of the reference,
// server/lorax_server/layers/tensor_parallel.py:193-250).  Each element crosses NVLink once in each direction per
// rank pair; at decode sizes (2 MB) the cost is two flag exchanges, not bandwidth.
//
// The grid is the same on every launch and every rank (blocks without elements still take part in A and C), so the
// flags simply carry the number of the launch, which is kept in a counter on the device (graph replays need no host
// input).  Every wait is bounded; on expiry the status word is set and the kernel leaves.
#include "common.cuh"

namespace lx {

constexpr int kArsBlocks = 64;
constexpr int kArsThreads = 512;
constexpr int kArsMaxRanks = 8;

struct ArSymParams {
  unsigned char* peers[kArsMaxRanks];   // base of every rank's symmetric buffer
  long long in_off, out_off, cnt_off;   // byte offsets inside the buffer; flags: int [2][kArsBlocks][kArsMaxRanks]
  int* epoch;                           // local: launches so far
  int* done;                            // local: blocks finished in this launch
  int rank, world;
  long long n_vec;                      // 16-byte vectors to reduce (tokens * hidden / 8)
  int* status;
  unsigned long long budget_ns;         // how long a block waits for a peer's flag before it gives up
};

// One flag per (stage, block, source rank), written with a release store by the source and polled with acquire loads by the
// owner: thread r of a block talks to rank r, so the `world` exchanges of a barrier run side by side.
LX_DEVICE void ars_post(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
LX_DEVICE int ars_peek(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
LX_DEVICE bool ars_wait(const int* p, int value, int* status, int where, unsigned long long budget_ns) {
  uint64_t t0 = 0;
  uint32_t polls = 0;
  while (true) {
    if (ars_peek(p) - value >= 0) return true;
    if ((++polls & 1023u) == 0) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) { report_status(status, kTimeoutPeerFlag, where); return false; }
    }
  }
}
// peer data: read past L1 (the acquire above orders it after the peer's writes)
LX_DEVICE uint4 ars_load(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// flags: int [2 stages][kArsBlocks][kArsMaxRanks]
LX_DEVICE int* ars_flag(unsigned char* base, long long cnt_off, int stage, int block, int src) {
  return reinterpret_cast<int*>(base + cnt_off) + (stage * kArsBlocks + block) * kArsMaxRanks + src;
}

// Barrier of block `b` with the same block on every rank.  Threads 0 .. world-1 each post to one rank and wait for that rank.
LX_DEVICE bool ars_barrier(const ArSymParams& p, int stage, int b, int value, int* ok_flag) {
  if (threadIdx.x == 0) *ok_flag = 1;
  __syncthreads();                      // also orders every thread's earlier stores before the posts (release is cumulative)
  if ((int)threadIdx.x < p.world) {
    const int r = threadIdx.x;
    ars_post(ars_flag(p.peers[r], p.cnt_off, stage, b, p.rank), value);
    if (!ars_wait(ars_flag(p.peers[p.rank], p.cnt_off, stage, b, r), value, p.status, 4000 + 1000 * stage + b, p.budget_ns)) *ok_flag = 0;
  }
  __syncthreads();
  return *ok_flag != 0;
}

template <int WORLD>
__global__ void __launch_bounds__(kArsThreads) allreduce_sym_kernel(const ArSymParams p) {
  __shared__ int ok_flag;
  const int b = blockIdx.x;
  const int epoch = *p.epoch;
  const int value = epoch + 1;
  constexpr int U = 8 / WORLD;          // vectors per thread and pass: eight 16-byte peer loads in flight whatever the group size
  if (ars_barrier(p, 0, b, value, &ok_flag)) {
    const long long v0 = p.n_vec * p.rank / WORLD, v1 = p.n_vec * (p.rank + 1) / WORLD;
    // a pass of a block covers U * 512 consecutive vectors; for a fixed u a warp reads 512 consecutive bytes
    for (long long pass = v0 + (long long)b * kArsThreads * U; pass < v1; pass += (long long)kArsBlocks * kArsThreads * U) {
      const long long base = pass + threadIdx.x;
      uint4 part[U][WORLD];
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int r = 0; r < WORLD; ++r) {
          if (base + u * kArsThreads < v1) part[u][r] = ars_load(p.peers[r] + p.in_off + (base + u * kArsThreads) * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (base + u * kArsThreads < v1) {
          float acc[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = 0.f;
#pragma unroll
          for (int r = 0; r < WORLD; ++r) {
            const uint32_t w[4] = {part[u][r].x, part[u][r].y, part[u][r].z, part[u][r].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = unpack_bf16x2(w[q]);
              acc[2 * q] += f.x;
              acc[2 * q + 1] += f.y;
            }
          }
          const uint4 res = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                                       pack_bf16x2(acc[6], acc[7]));
#pragma unroll
          for (int r = 0; r < WORLD; ++r) *reinterpret_cast<uint4*>(p.peers[r] + p.out_off + (base + u * kArsThreads) * 16) = res;
        }
      }
    }
    ars_barrier(p, 1, b, value, &ok_flag);
  }
  if (threadIdx.x == 0) {
    // the last block of the launch advances the launch counter (every block has read it by now)
    __threadfence();
    if (atomicAdd(p.done, 1) == (int)gridDim.x - 1) {
      *p.done = 0;
      *p.epoch = epoch + 1;
    }
  }
}

}  // namespace lx

extern "C" {

int lx_allreduce_sym_blocks() { return lx::kArsBlocks; }

// How long the kernels that wait for another GPU (this all-reduce, the GEMM + all-reduce) poll a peer's flag before they set
// the status word and return.  Applies to launches made after the call; 0 restores the default of two seconds.
void lx_set_wait_budget_ns(unsigned long long ns) { lx::host_wait_budget_ns() = ns ? ns : lx::kWaitBudgetNs; }
unsigned long long lx_get_wait_budget_ns() { return lx::host_wait_budget_ns(); }

// Bytes of the flag area (2 stages x blocks x 8 ranks ints) a rank must zero once before the first launch.
int lx_allreduce_sym_counter_bytes() { return 2 * lx::kArsBlocks * lx::kArsMaxRanks * 4; }

// In-place semantics across the group: input areas hold every rank's partial [n_elems] bf16, afterwards every rank's
// output area holds the sum.  `state` points at two zero-initialised local ints (launch counter, finished blocks).
int lx_allreduce_sym(const unsigned long long* peer_ptrs, int rank, int world, long long in_off, long long out_off, long long cnt_off,
                     long long n_elems, int* state, int* status, void* stream) {
  using namespace lx;
  if (n_elems <= 0) return 0;
  if ((world != 2 && world != 4 && world != 8) || (n_elems % 8) != 0 || ((in_off | out_off) % 16) != 0) return -1;
  ArSymParams p{};
  for (int r = 0; r < world; ++r) p.peers[r] = reinterpret_cast<unsigned char*>(peer_ptrs[r]);
  p.in_off = in_off; p.out_off = out_off; p.cnt_off = cnt_off;
  p.epoch = state; p.done = state + 1;
  p.rank = rank; p.world = world; p.n_vec = n_elems / 8; p.status = status;
  p.budget_ns = host_wait_budget_ns();
  // all blocks of all ranks wait on one another: 64 blocks of 512 threads are always co-resident on a B200
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (world == 2) allreduce_sym_kernel<2><<<kArsBlocks, kArsThreads, 0, s>>>(p);
  else if (world == 4) allreduce_sym_kernel<4><<<kArsBlocks, kArsThreads, 0, s>>>(p);
  else allreduce_sym_kernel<8><<<kArsBlocks, kArsThreads, 0, s>>>(p);
  return -(int)cudaGetLastError();
}

}  // extern "C"
