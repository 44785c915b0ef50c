// Work distribution shared by the tcgen05 GEMM kernels ("stream-K").
//
// A worker is a persistent CTA (or CTA pair).  The first sk_tiles output tiles are cut along K into
// one equal, contiguous range of k-blocks per worker; the remaining tiles are handed out whole,
// round-robin, after that.  A worker whose range starts inside a tile computes a partial tile: it
// writes it (fp32) to its own workspace slot and raises the tile's arrival counter.  The worker that
// owns the tile's first k-blocks - the last piece of its own range, so the others are done long
// before - adds the partials in worker order and runs the epilogue.  The order of the sum is fixed, so
// results do not depend on timing.
#pragma once
#include "tc05.cuh"

namespace tfb {

constexpr int kFlagBytes = 8192;  // head of the workspace: arrival counters, zero between kernels

struct Segments {
  int kblocks, tiles, workers;
  int64_t it, hi;  // cursor and end of this worker's k-block range in the split region
  int next_tile;   // next whole tile
  __device__ Segments(int kblocks_, int tiles_, int sk_tiles, int workers_, int worker, bool dead) {
    kblocks = kblocks_;
    tiles = dead ? 0 : tiles_;
    workers = workers_;
    const int64_t sk_iters = dead ? 0 : (int64_t)sk_tiles * kblocks;
    it = sk_iters * worker / workers;
    hi = sk_iters * (worker + 1) / workers;
    next_tile = sk_tiles + worker;
  }
  // Next segment: k-blocks [kb0, kb1) of `tile`.  kb0 > 0: a partial to hand over; kb0 == 0 and
  // kb1 < kblocks: the part that collects the others; otherwise a whole tile.
  __device__ bool next(int& tile, int& kb0, int& kb1) {
    if (it < hi) {
      tile = (int)(it / kblocks);
      kb0 = (int)(it % kblocks);
      const int64_t left = hi - it;
      kb1 = (left < kblocks - kb0) ? kb0 + (int)left : kblocks;
      it += kb1 - kb0;
      return true;
    }
    if (next_tile < tiles) {
      tile = next_tile;
      kb0 = 0;
      kb1 = kblocks;
      next_tile += workers;
      return true;
    }
    return false;
  }
};

// Number of workers after `worker` whose ranges reach into `tile` (their partials are added by it).
__device__ __forceinline__ int partials_expected(int tile, int kblocks, int sk_tiles, int workers, int worker) {
  const int64_t sk_iters = (int64_t)sk_tiles * kblocks;
  const int64_t tile_end = (int64_t)(tile + 1) * kblocks;
  int c = worker + 1;
  while (c < workers && sk_iters * c / workers < tile_end) ++c;
  return c - worker - 1;
}

// Bounded wait until *flag reaches `expect` (acquire).  Same limit and status word as mbar_wait.
__device__ __forceinline__ bool flag_wait(const int* flag, int expect, int code, volatile int* abort_flag) {
  const uint64_t t0 = global_ns();
  for (;;) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= expect) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > kWaitLimitNs) break;
    __nanosleep(64);
  }
  *abort_flag = 1;
  atomicCAS(&g_dev_status, 0, code);
  return false;
}

}  // namespace tfb
