// q8_group_tok for short rows (512 columns: a down projection's), a thread a row.
//
// The contract's sums, computed where no value has to move: with 512 columns a row has 16 blocks, one for each of the
// contract's 16 lanes, so "lane l's chain" is the single product fmaf(d_x[l], block_l, 0) and the xor tree adds the
// sixteen of them in a fixed pairing - (l, l ^ 8), then (l, l ^ 4), (l, l ^ 2), (l, l ^ 1). One thread that holds
// all sixteen products makes the same additions in registers, with no shuffle and no second pass. It also decodes
// whole superblocks, so every byte offset is a compile-time constant (a row of two 2-mod-4-byte superblocks starts
// on a word: the first superblock is aligned, the second starts mid-word).
//
// A warp is 32 consecutive rows. Its tokens' int8 rows (one or two tokens a task) sit in the warp's own piece of
// shared memory, read by all 32 threads at the same address (a broadcast); the weights come by bulk copies into the
// warp's own two slots, as in lane_ring.cu, and the block never meets after its start-up.
#include "lane_rows_api.h"

#include "dispatch.cuh"
#include "lane_staged.cuh"

namespace osmos {
namespace rows {
namespace {

using namespace tma;
using staged::build_luts;
using staged::Rep;
using staged::RepLuts2;
using staged::build_luts2;
using staged::Super;

constexpr int kWarps = 12, kThreads = kWarps * kWarp;
constexpr int kSlots = 2;
constexpr int kNT = 2;
constexpr int kNSB = 2, kCols = kNSB * 256, kBlocks = kCols / 32;  // the one shape: 512 columns, 16 blocks
constexpr uint32_t kMaxEntries = 1024;
constexpr uint32_t kSmemLimit = 226u * 1024u;
constexpr uint32_t kXBytes = kNT * (kCols + kBlocks * 4);  // a warp's activations: int8 rows, then their scales

__device__ uint32_t g_status;

struct Args {
  const uint8_t* const* w;
  const int32_t *cnt, *xrow, *xin;
  const int8_t* q;
  const float* d;
  float* out;
  uint32_t rows, out_stride, n_entries, max_cnt;
  uint32_t list_off, ptr_off, x_off, ring_off, slot_bytes;
  uint32_t* status;
  LaneEp ep;
};

template <uint32_t T>
__global__ void __launch_bounds__(kThreads, 1) lane_rows_kernel(const Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[kWarps][kSlots];
  __shared__ int s_scan[kWarps];
  __shared__ int s_pairs;
  constexpr int SB = Super<T>::bytes;
  constexpr uint32_t row_bytes = kNSB * SB;
  static_assert(row_bytes % 4 == 0, "a row starts on a word");
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  uint16_t* list = (uint16_t*) (smem + a.list_off);
  const uint8_t** wptr = (const uint8_t**) (smem + a.ptr_off);
  int2* meta = (int2*) (wptr + a.n_entries);  // an entry's (live tokens, first row): no trip to the tables a task
  uint8_t* xs = smem + a.x_off + warp * kXBytes;
  uint8_t* ring = smem + a.ring_off + warp * kSlots * a.slot_bytes;

  if (lane == 0) {
    for (int s = 0; s < kSlots; s++) bar_init(&full[warp][s], 1);
    bar_init_fence();
  }
  const RepLuts2<T> luts = build_luts2<T>(smem, kThreads);
  // (a dependent launch: the tables and activations read from here on may be the output of the kernels ahead; the
  // codebooks above are not)
  pdl_wait();
  pdl_launch_next();
  // (the expert-parallel step: inputs of an odd step in the buffers' second halves, rows stored where a table says)
  const uint32_t parity = a.ep.step ? (*a.ep.step & 1u) : 0u;
  const int8_t* const in_q = a.q + parity * a.ep.half_q;
  const float* const in_d = (const float*) ((const uint8_t*) a.d + parity * a.ep.half_d);

  auto live_count = [&](uint32_t m) -> uint32_t {
    const int32_t c = a.cnt[m];
    return c <= 0 ? 0u : ((uint32_t) c < a.max_cnt ? (uint32_t) c : a.max_cnt);
  };
  bool aligned = true;
  {
    uint32_t run = 0;
    for (uint32_t base = 0; base < a.n_entries; base += kThreads) {
      const uint32_t m = base + tid;
      uint32_t mine = 0;
      if (m < a.n_entries) {
        const uint32_t c = live_count(m);
        meta[m] = make_int2((int) c, a.xrow[m]);
        mine = (c + kNT - 1) / kNT;
        const uint8_t* g = a.w[m];
        wptr[m] = g;
        if (mine && ((uintptr_t) g & 15u)) aligned = false;
      }
      uint32_t inc = mine;
#pragma unroll
      for (int o = 1; o < kWarp; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o, kWarp);
        if (lane >= (uint32_t) o) inc += up;
      }
      if (lane == kWarp - 1) s_scan[warp] = (int) inc;
      __syncthreads();
      uint32_t before = run, all = 0;
      for (uint32_t wv = 0; wv < (uint32_t) kWarps; wv++) {
        if (wv < warp) before += (uint32_t) s_scan[wv];
        all += (uint32_t) s_scan[wv];
      }
      const uint32_t pos = before + inc - mine;
      for (uint32_t gq = 0; gq < mine; gq++) list[pos + gq] = (uint16_t) (m | gq << 10);
      run += all;
      __syncthreads();
    }
    if (tid == 0) s_pairs = (int) run;
  }
  const int any_bad = __syncthreads_or(aligned ? 0 : 1);
  if (any_bad) {  // a matrix that is not 16-byte aligned cannot be copied in bulk: the launch stands down
    if (tid == 0) atomicOr(a.status, 2u);
    return;
  }
  const uint32_t tpp = a.rows / kWarp;  // tasks an (entry, token group): 32 rows each
  const uint32_t tasks = (uint32_t) s_pairs * tpp;
  // (a block's warps take neighbouring tasks: mostly the same entry and tokens, whose activations then come from L1)
  const uint32_t gw = blockIdx.x * kWarps + warp, stride = gridDim.x * kWarps;

  auto issue = [&](uint32_t n) {  // one lane: the warp's n-th task into slot n % kSlots
    const uint32_t tk = gw + n * stride;
    if (tk >= tasks) return;
    const uint32_t pair = tk / tpp, row0 = (tk - pair * tpp) * kWarp;
    const uint32_t m = list[pair] & 0x3FFu, slot = n % kSlots;
    bar_expect(&full[warp][slot], a.slot_bytes);
    bulk_load(ring + slot * a.slot_bytes, wptr[m] + (uint64_t) row0 * row_bytes, a.slot_bytes, &full[warp][slot]);
  };
  if (lane == 0)
    for (uint32_t n = 0; n < (uint32_t) kSlots; n++) issue(n);

  const uint32_t xsa = smem_addr(xs);
  // one superblock (alignment A) of this thread's row: its eight blocks' products into prod[8 i ...]
  auto superblock = [&](auto align_tag, auto live_tag, uint32_t src, int i, float (*prod)[kBlocks]) {
    constexpr int A = decltype(align_tag)::value, NTL = decltype(live_tag)::value;
    WordWindow<Super<T>::words, A> win;
#pragma unroll
    for (int k = 0; k < Super<T>::words; k++) win.w[k] = lds32(src - A + 4 * k);
#pragma unroll
    for (int j = 0; j < 8; j++) {
      LaneCodes c;
      lane_codes_rd<T>(win, j, c, luts);
#pragma unroll
      for (int t = 0; t < NTL; t++) {
        const uint32_t xa = xsa + (uint32_t) t * kCols + (uint32_t) (8 * i + j) * 32u;
        const int4 lo = lds128(xa), hi = lds128(xa + 16);
        const int x[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const float dx = ldsf(xsa + kNT * kCols + ((uint32_t) t * kBlocks + 8 * i + j) * 4u);
        prod[t][8 * i + j] = __fmaf_rn(dx, lane_block_sum<T>(c, x), 0.0f);
      }
    }
  };
  auto do_task = [&](auto live_tag, uint32_t sa, uint32_t row, float* const (&orow)[kNT]) {
    constexpr int NTL = decltype(live_tag)::value;
    using A0 = std::integral_constant<int, 0>;
    using A2 = std::integral_constant<int, (SB % 4) ? 2 : 0>;
    float prod[NTL][kBlocks];
    const uint32_t ra = sa + lane * row_bytes;
    superblock(A0{}, live_tag, ra, 0, prod);
    superblock(A2{}, live_tag, ra + SB, 1, prod);
#pragma unroll
    for (int t = 0; t < NTL; t++) {
#pragma unroll
      for (int o = kBlocks / 2; o > 0; o >>= 1)
#pragma unroll
        for (int l = 0; l < o; l++) prod[t][l] = __fadd_rn(prod[t][l], prod[t][l + o]);
      orow[t][row] = prod[t][0];
    }
  };

  using I1 = std::integral_constant<int, 1>;
  using I2 = std::integral_constant<int, kNT>;
  // a task's tokens: this lane's 16 bytes of each int8 row and, on the first sixteen lanes, a block scale - read a task
  // ahead into registers, so that the trip to L2 runs under the task before
  auto fetch = [&](uint32_t n, int4 (&xq)[kNT], float (&xd)[kNT]) {
    const uint32_t tk = gw + n * stride;
    if (tk >= tasks) return;
    const uint32_t v = list[tk / tpp], g = v >> 10;
    const int2 me = meta[v & 0x3FFu];
    const uint32_t left = (uint32_t) me.x - g * kNT, r0 = (uint32_t) me.y + g * kNT;
#pragma unroll
    for (int t = 0; t < kNT; t++)
      if ((uint32_t) t < left) {
        const uint32_t r = r0 + t;
        const uint64_t xr = a.xin ? (uint64_t) (uint32_t) a.xin[r] : r;
        xq[t] = __ldg((const int4*) (in_q + xr * kCols) + lane);
        if (lane < (uint32_t) kBlocks) xd[t] = __ldg(in_d + xr * kBlocks + lane);
      }
  };
  int4 xq[kNT];
  float xd[kNT];
#pragma unroll
  for (int t = 0; t < kNT; t++) xq[t] = make_int4(0, 0, 0, 0), xd[t] = 0.0f;
  fetch(0, xq, xd);
  for (uint32_t n = 0;; n++) {
    const uint32_t tk = gw + n * stride;
    if (tk >= tasks) break;
    const uint32_t pair = tk / tpp, row0 = (tk - pair * tpp) * kWarp;
    const uint32_t v = list[pair], m = v & 0x3FFu, g = v >> 10;
    const int2 me = meta[m];
    const uint32_t cnt = (uint32_t) me.x, live = cnt - g * kNT < (uint32_t) kNT ? cnt - g * kNT : (uint32_t) kNT;
    const uint32_t r0 = (uint32_t) me.y + g * kNT;
    // the task's tokens into the warp's piece of shared memory: 16 bytes a lane a token, then the scales
    __syncwarp();  // (every lane has finished the last task's reads)
    float* orow[kNT];  // where each token's results go: looked up now, used when the task's rows are done
#pragma unroll
    for (int t = 0; t < kNT; t++) {
      const uint32_t ro = r0 + ((uint32_t) t < live ? (uint32_t) t : live - 1);
      orow[t] = a.ep.out_rows ? a.ep.out_rows[ro] : a.out + (uint64_t) ro * a.out_stride;
      if ((uint32_t) t < live) {
        ((int4*) (xs + t * kCols))[lane] = xq[t];
        if (lane < (uint32_t) kBlocks) ((float*) (xs + kNT * kCols))[t * kBlocks + lane] = xd[t];
      }
    }
    __syncwarp();
    fetch(n + 1, xq, xd);
    const uint32_t slot = n % kSlots;
    if (!bar_wait(&full[warp][slot], (n / kSlots) & 1u)) {  // a copy never landed: report it and leave
      if (lane == 0) atomicOr(a.status, 1u);
      break;
    }
    const uint32_t sa = smem_addr(ring + slot * a.slot_bytes);
    if (live == (uint32_t) kNT) do_task(I2{}, sa, row0 + lane, orow);
    else do_task(I1{}, sa, row0 + lane, orow);
    __syncwarp();  // every lane is done reading the slot: refill it
    if (lane == 0) {
      fence_async_smem();
      issue(n + kSlots);
    }
  }
  if (a.ep.publish)  // (every thread of every block comes here: a block that stood down above has left already)
    publish_step(a.ep.peers, a.ep.flags_off, a.ep.rank, a.ep.n_ranks, *a.ep.step, a.ep.counter, nullptr);
}

struct Device {
  int sms = 0, index = 0;
  uint32_t* status = nullptr;
};

const Device* device_info() {
  static Device devs[64];
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
  if (!devs[d].status) {
    void* at = nullptr;
    int sms = 0;
    if (cudaGetSymbolAddress(&at, g_status) != cudaSuccess || !at) return nullptr;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || sms <= 0) return nullptr;
    devs[d].sms = sms, devs[d].index = d, devs[d].status = (uint32_t*) at;
  }
  return &devs[d];
}

template <uint32_t T>
int launch(const Request& r, cudaStream_t s) {
  const Device* dev = device_info();
  if (!dev) return 0;
  Args a{};
  a.list_off = (uint32_t) ((Rep<T>::bytes + 127) & ~127);
  a.ptr_off = a.list_off + kMaxEntries * (8 / kNT) * 2;
  a.x_off = (a.ptr_off + r.n_entries * 16 + 127u) & ~127u;  // (pointers, then (count, first row))
  a.ring_off = (a.x_off + kWarps * kXBytes + 127u) & ~127u;
  a.slot_bytes = kWarp * kNSB * Super<T>::bytes;
  const uint32_t total = a.ring_off + kWarps * kSlots * a.slot_bytes + 16u;
  if (total > kSmemLimit) return 0;
  a.w = (const uint8_t* const*) r.w, a.cnt = r.cnt, a.xrow = r.xrow, a.xin = r.xin, a.q = r.q, a.d = r.d, a.out = r.out;
  a.rows = r.rows, a.out_stride = r.out_stride, a.n_entries = r.n_entries, a.max_cnt = r.max_cnt;
  a.status = dev->status;
  a.ep = r.ep;
  if (r.dry) return 1;
  static bool sized[64] = {};  // (per template instance and device: the attribute belongs to a device's context)
  auto kernel = lane_rows_kernel<T>;
  if (!allow_dynamic_smem(kernel, (int) kSmemLimit, sized)) return 0;
  return launch_dependent(kernel, dim3((uint32_t) dev->sms), dim3(kThreads), total, s, a) == cudaSuccess ? 1 : -1;
}

}  // namespace

int try_launch(uint32_t type, const Request& r, void* stream) {
  if (r.cols != (uint32_t) kCols || !r.rows || r.rows % kWarp || !r.n_entries || r.n_entries > kMaxEntries) return 0;
  if (!r.max_cnt || r.max_cnt > 8 || ((uintptr_t) r.q & 15u) || ((uintptr_t) r.d & 3u)) return 0;
  const cudaStream_t s = (cudaStream_t) stream;
  switch (type) {
    case QTYPE_IQ3_XXS: return launch<QTYPE_IQ3_XXS>(r, s);
    case QTYPE_IQ2_XXS: return launch<QTYPE_IQ2_XXS>(r, s);
    case QTYPE_IQ1_S: return launch<QTYPE_IQ1_S>(r, s);
    case QTYPE_IQ1_M: return launch<QTYPE_IQ1_M>(r, s);
    default: return 0;
  }
}

uint32_t read_status() {
  const Device* dev = device_info();
  if (!dev) return 0x80000000u;
  uint32_t v = 0, zero = 0;
  if (cudaMemcpy(&v, dev->status, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return 0x80000000u;
  cudaMemcpy(dev->status, &zero, sizeof zero, cudaMemcpyHostToDevice);
  return v;
}

}  // namespace rows
}  // namespace osmos
