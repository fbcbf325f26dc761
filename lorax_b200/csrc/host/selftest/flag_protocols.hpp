// CPU-thread models of the two device-side synchronisation protocols, run under ThreadSanitizer by the host self test.
//
// The kernels themselves cannot run under a race detector, so the protocols are restated here with std::atomic (same orders:
// release stores / acquire loads, relaxed counters where the kernels use them) around PLAIN data arrays.  A thread plays a
// CUDA block; the data a block reads after a wait is written by another block before its post, exactly as on the device, so a
// missing or misplaced wait shows up as a data race or as a wrong sum.
//
//   model_all_reduce   csrc/kernels/allreduce_sym.cu: per (stage, block, source rank) flags carrying the launch number, every
//                      rank reduces its slice from all ranks' inputs and stores it to all ranks' outputs, second flag round,
//                      the last block of a launch advances the launch counter.  Ranks run their launches independently: a
//                      rank may be one launch ahead of its peers.
//   model_lora_sync    csrc/kernels/gemm_bf16.cu (LoRA inside the GEMM launch): CTAs first produce "images" (with K splits
//                      handed over through arrival counters, the last arrival writes), count themselves in, and consumers
//                      read images only after every CTA of the launch has; the last CTA to finish clears the counters.
#pragma once

#include <atomic>
#include <cstdint>
#include <thread>
#include <vector>

namespace lx_model {

inline bool model_all_reduce(int world, int blocks, int n, int launches) {
  struct Rank {
    std::vector<float> in, out;
    std::vector<std::atomic<int>> flags;      // [2][blocks][world]
    std::atomic<int> epoch{0}, done{0};
    Rank(int n, int blocks, int world) : in(n), out(n), flags(2 * blocks * world) { for (auto& f : flags) f.store(0); }
  };
  std::vector<std::unique_ptr<Rank>> ranks;
  for (int r = 0; r < world; ++r) ranks.emplace_back(new Rank(n, blocks, world));
  std::atomic<bool> bad{false};
  auto flag = [&](int rank, int stage, int b, int src) -> std::atomic<int>& { return ranks[rank]->flags[(stage * blocks + b) * world + src]; };
  auto barrier = [&](int me, int stage, int b, int value) {
    for (int r = 0; r < world; ++r) flag(r, stage, b, me).store(value, std::memory_order_release);
    for (int r = 0; r < world; ++r)
      while (flag(me, stage, b, r).load(std::memory_order_acquire) - value < 0) std::this_thread::yield();
  };
  auto rank_main = [&](int me) {
    Rank& R = *ranks[me];
    for (int l = 0; l < launches; ++l) {
      for (int i = 0; i < n; ++i) R.in[i] = (float)((i * 7 + l * 3 + me) % 11);        // the producer kernel of this launch
      std::vector<std::thread> blk;
      for (int b = 0; b < blocks; ++b) blk.emplace_back([&, b] {
        const int value = R.epoch.load(std::memory_order_relaxed) + 1;
        barrier(me, 0, b, value);
        const int v0 = n * me / world, v1 = n * (me + 1) / world;
        for (int i = v0 + b; i < v1; i += blocks) {
          float acc = 0.f;
          for (int r = 0; r < world; ++r) acc += ranks[r]->in[i];
          for (int r = 0; r < world; ++r) ranks[r]->out[i] = acc;
        }
        barrier(me, 1, b, value);
        if (R.done.fetch_add(1, std::memory_order_acq_rel) == blocks - 1) {
          R.done.store(0, std::memory_order_relaxed);
          R.epoch.store(value, std::memory_order_release);
        }
      });
      for (auto& t : blk) t.join();
      for (int i = 0; i < n; ++i) {                                                      // the consumer kernel of this launch
        float want = 0.f;
        for (int r = 0; r < world; ++r) want += (float)((i * 7 + l * 3 + r) % 11);
        if (R.out[i] != want) bad.store(true);
      }
    }
  };
  std::vector<std::thread> ts;
  for (int r = 0; r < world; ++r) ts.emplace_back(rank_main, r);
  for (auto& t : ts) t.join();
  return !bad.load();
}

inline bool model_lora_sync(int ctas, int items, int ksplit, int launches) {
  std::vector<int> image(items, 0);                 // plain data: the operand images
  std::vector<int> partial(items * ksplit, 0);      // plain data: K-split partials
  std::vector<std::atomic<int>> counters(items);
  for (auto& c : counters) c.store(0);
  std::atomic<int> finished{0}, shrunk{0};
  std::atomic<bool> bad{false};
  for (int l = 0; l < launches; ++l) {
    std::vector<std::thread> ts;
    for (int c = 0; c < ctas; ++c) ts.emplace_back([&, c] {
      // shrink items of this CTA (item, split) pairs dealt round-robin
      for (int idx = c; idx < items * ksplit; idx += ctas) {
        const int it = idx / ksplit, sp = idx % ksplit;
        partial[it * ksplit + sp] = (l + 1) * 100 + it + sp;
        if (counters[it].fetch_add(1, std::memory_order_acq_rel) == ksplit - 1) {      // last arrival adds the partials up
          counters[it].store(0, std::memory_order_relaxed);
          int sum = 0;
          for (int q = 0; q < ksplit; ++q) sum += partial[it * ksplit + q];
          image[it] = sum;
        }
      }
      shrunk.fetch_add(1, std::memory_order_release);
      // base tiles: the first one that needs an image waits for every CTA of the launch
      while (shrunk.load(std::memory_order_acquire) != ctas) std::this_thread::yield();
      for (int it = c % 3; it < items; it += 3) {
        int want = 0;
        for (int q = 0; q < ksplit; ++q) want += (l + 1) * 100 + it + q;
        if (image[it] != want) bad.store(true);
      }
      if (finished.fetch_add(1, std::memory_order_acq_rel) == ctas - 1) {               // the last CTA clears the counters
        finished.store(0, std::memory_order_relaxed);
        shrunk.store(0, std::memory_order_release);
      }
    });
    for (auto& t : ts) t.join();                                                         // kernel boundary
    if (finished.load() != 0 || shrunk.load() != 0) bad.store(true);
    for (auto& c : counters) if (c.load() != 0) bad.store(true);
  }
  return !bad.load();
}

}  // namespace lx_model
