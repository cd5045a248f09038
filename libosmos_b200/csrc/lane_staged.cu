// Host side of the int8 lane's staged kernel (lane_staged.cuh): which shapes it takes, its tile size and shared-memory
// plan, and the launch. q8.cu's entry points try it first and fall back to the generic kernel for the shapes it
// does not take - the two give the same bits.
#include "lane_staged.cuh"

#include "dispatch.cuh"
#include "lane_staged_api.h"

namespace osmos {
namespace staged {
namespace {

constexpr uint32_t kSmemLimit = 226u * 1024u;  // dynamic; the block also has a few static words (227 KB in all a block)

__device__ uint32_t g_status;

struct Device {
  int sms = 0;
  uint32_t* status = nullptr;
};

// the current device's SM count and the device address of its status word, looked up once per device
const Device* device_info() {
  static Device devs[64];
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
  if (!devs[d].status) {
    void* at = nullptr;
    int sms = 0;
    if (cudaGetSymbolAddress(&at, g_status) != cudaSuccess || !at) return nullptr;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || sms <= 0) return nullptr;
    devs[d].sms = sms, devs[d].status = (uint32_t*) at;
  }
  return &devs[d];
}

template <uint32_t T, bool FUSED, bool DENSE>
int launch(const Request& r, cudaStream_t s) {
  const Device* dev = device_info();
  if (!dev) return 0;
  constexpr int M = FUSED ? 2 : 1;
  const uint32_t row_bytes = r.cols / 256 * Super<T>::bytes;
  // a tile's rows: as many as one pass of the compute warps covers (phase A: a thread a superblock of one matrix), in
  // eights; the light one-scale blocks take half a pass, so that more stages are in flight
  const uint32_t nsb = r.cols / 256, pass = (FUSED ? kComputeThreads / 2 : kComputeThreads) / (kLanePlain<T> ? 2 : 1);
  uint32_t tr = (pass / nsb) & ~7u;
  if (tr > r.rows) tr = r.rows;
  if (tr < 8) tr = 8;
  if (DENSE)  // a small matrix: enough tiles that every block has a few to pipeline
    while (tr > 8 && (uint64_t) ((r.rows + tr - 1) / tr) * ((r.n_tok + kNT - 1) / kNT) < 4ull * dev->sms) tr -= 8;
  while (tr > 8 && make_plan<T>(r.cols, tr, M, 2).total > kSmemLimit) tr -= 8;
  if (make_plan<T>(r.cols, tr, M, 2).total > kSmemLimit) return 0;
  uint32_t stages = 2;  // as deep a ring as shared memory holds
  while (stages < (uint32_t) kMaxStages && make_plan<T>(r.cols, tr, M, stages + 1).total <= kSmemLimit) stages++;
  const Plan p = make_plan<T>(r.cols, tr, M, stages);
  static bool sized[64] = {};  // (one record a template instance, one flag a device)
  auto kernel = lane_staged_kernel<T, FUSED, DENSE>;
  if (!allow_dynamic_smem(kernel, (int) kSmemLimit, sized)) return 0;
  Args a{};
  a.w_dense = (const uint8_t*) r.w_dense, a.wg = (const uint8_t* const*) r.wg, a.wu = (const uint8_t* const*) r.wu;
  a.cnt = r.cnt, a.xrow = r.xrow, a.xin = r.xin, a.win = r.win, a.q = r.q, a.d = r.d, a.scale = r.scale, a.lim = r.lim;
  a.out = r.out, a.rows = r.rows, a.cols = r.cols, a.out_stride = r.out_stride, a.n_entries = r.n_entries;
  a.max_cnt = DENSE ? r.n_tok : r.max_cnt, a.n_tok = r.n_tok, a.tile_rows = tr, a.tiles = (r.rows + tr - 1) / tr;
  a.stages = stages;
  a.status = dev->status;
  uint32_t grid = (uint32_t) dev->sms;
  if (DENSE) {
    const uint64_t items = (uint64_t) a.tiles * ((r.n_tok + kNT - 1) / kNT);
    if (items < grid) grid = (uint32_t) items;
  }
  kernel<<<grid, kThreads, p.total, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace

int try_launch(uint32_t type, const Request& r, void* stream) {
  // shapes the staged kernel takes: whole 256-value superblocks, rows in eights (so every tile's bytes are a multiple
  // of 16), 16-byte aligned activations, few enough superblocks a row for the tables' 12-bit fields
  if (r.cols % 256 || r.rows % 8 || r.cols / 256 > 256) return 0;
  if (((uintptr_t) r.q | (uintptr_t) r.d | (uintptr_t) r.w_dense) & 15u) return 0;
  if (r.dense && r.n_tok > 8) return 0;
  const cudaStream_t s = (cudaStream_t) stream;
#define CASE(T)                                                  \
  if (r.dense) return launch<T, false, true>(r, s);              \
  if constexpr (!kLanePlain<T>) {                                \
    if (r.fused) return launch<T, true, false>(r, s);            \
    return launch<T, false, false>(r, s);                        \
  }                                                              \
  return 0;
  OSMOS_SWITCH_LANE_EXT(type, CASE, return 0)
#undef CASE
}

uint32_t read_status() {
  const Device* dev = device_info();
  if (!dev) return 0x80000000u;
  uint32_t v = 0, zero = 0;
  if (cudaMemcpy(&v, dev->status, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return 0x80000000u;
  cudaMemcpy(dev->status, &zero, sizeof zero, cudaMemcpyHostToDevice);
  return v;
}

}  // namespace staged
}  // namespace osmos
