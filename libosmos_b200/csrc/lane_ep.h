// What the expert-parallel step adds to a launch of the warp-ring and thread-a-row lane kernels (all of it optional):
// inputs that alternate between two halves by the step's parity, outputs that go row by row to addresses from a table
// (a row's place in its token's home rank, written over NVLink by plain stores), and the release of this rank's flag in
// every rank's buffer once the last row is stored.
#pragma once
#include <cstdint>

#include "ep_sync.cuh"

namespace osmos {

struct LaneEp {
  const uint32_t* step = nullptr;  // the step counter (device); NULL: no parity, nothing published
  uint64_t half_q = 0, half_d = 0, half_scale = 0;  // an odd step's q / d / scale lie this many bytes further
  float* const* out_rows = nullptr;  // row r's results at out_rows[r][matrix row] instead of out + r * stride
  bool publish = false;              // after the last store: the step into flags_off + 4 * rank of every rank's buffer
  EpPeers peers = {};
  uint64_t flags_off = 0;
  uint32_t rank = 0, n_ranks = 0;
  uint32_t* counter = nullptr;       // a zeroed device word the publishing kernel uses and leaves zero
};

}  // namespace osmos
