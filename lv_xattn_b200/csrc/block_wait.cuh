// Host-side translation of the ABI's lvx_block_wait into the kernels' BlockWait (see sm100_prims.cuh).
#pragma once
#include "lvx_internal.h"
#include "sm100_prims.cuh"

namespace lvx {

inline BlockWait make_block_wait(const lvx_block_wait* w, int q_blocks) {
  BlockWait b;
  b.flags = nullptr;
  b.epoch = 0;
  b.first_blk = 0;
  b.limit = 0;
  b.pipe_limit = LVX_SPIN_LIMIT_CYCLES;
  if (w != nullptr && w->my_flags != nullptr) {
    b.flags = w->my_flags + size_t(w->slot) * LVX_MAX_PEERS;
    b.epoch = w->epoch;
    b.first_blk = w->first_block;
    b.limit = p2p_wait_limit_cycles();
    b.pipe_limit = LVX_SPIN_LIMIT_CYCLES + b.limit;
  } else if (w != nullptr) {
    b.first_blk = w->first_block;      // block order only, nothing to wait for
  }
  if (b.first_blk < 0 || b.first_blk >= q_blocks) b.first_blk = 0;
  return b;
}

}  // namespace lvx
