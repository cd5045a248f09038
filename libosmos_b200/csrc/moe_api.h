// what the expert-parallel step (ep.cu) asks of the lane tables (moe.cu): the same tables, built after a bounded wait
// on the peers' dispatch flags, with each row's place in its home rank's receive block
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "ep_sync.cuh"
#include "osmos_b200/lane.h"

namespace osmos {

struct LaneTablesSync {
  const uint32_t* flags = nullptr;  // this rank's dispatch flags, a word a sender (NULL: no wait)
  const uint32_t* step = nullptr;   // the step counter (device): the value the flags must have reached
  uint32_t n_ranks = 0;
  uint64_t half_bytes = 0;          // an odd step's ids lie this many bytes after the even steps'
  const float* weights = nullptr;   // the picks' routed weights (an even step's; an odd step's weights_half bytes on)
  uint64_t weights_half = 0;
  uint32_t* status = nullptr;       // bit 0 set when a wait ran out
};

struct LaneRowHomes {
  float** rows = nullptr;  // out [picks]: where row r's result goes (NULL: not wanted)
  float* scale = nullptr;  // out [picks]: row r's routed weight (NULL: not wanted) - a row's gate / up scale without the
                           // trip through its pick index
  uint8_t* base[16] = {};  // every rank's exchange buffer as mapped here
  uint64_t recv[2] = {};   // the receive block's offset in a buffer, by step parity
  uint32_t tokens = 0;     // home tokens a rank
  uint32_t dim = 0;
};

bool lane_tables_launch(const int32_t* ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t expert0, uint32_t expert1,
                        const LaneExperts* ex, const LaneTables* t, const LaneTablesSync& sy, const LaneRowHomes& homes,
                        cudaStream_t s);

}  // namespace osmos
