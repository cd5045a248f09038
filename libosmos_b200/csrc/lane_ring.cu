// The int8 lane's grouped entry points (q8_gate_up, q8_group_tok) with every warp working alone.
//
// The sums are the contract's: a row's 32-value blocks go to L = 16 lanes (32 from 4096 columns), lane l taking
// blocks l, l + L, ... in order with one fmaf a block, then the xor tree over the L lanes (decode.cuh has the
// arithmetic of a block). What this kernel changes is who does the work when:
//   - a warp is a row's L lanes (two rows at once when L is 16: a gate row and its up row for q8_gate_up, two rows
//     of the matrix for q8_group_tok), so a row's chain and tree stay in registers and no value crosses warps;
//   - the int8 activations of the lane's blocks, for up to two tokens, sit in registers for a whole task (a run of
//     rows of one entry), loaded while the task's first weights are still on their way;
//   - the weights come by bulk copies into a ring of slots that belongs to the warp: it waits on its own mbarriers,
//     and refills a slot the moment its lanes have read it. After the start-up (codebooks, the list of live entries,
//     their matrix pointers) the block never meets again.
// Tasks are dealt round-robin to all warps of the grid in (entry, rows) order, block by block (task i to block
// i % blocks), so the blocks' shares differ by one task at most.
#include "lane_ring_api.h"

#include "dispatch.cuh"
#include "lane_staged.cuh"
#include "lane_warp.cuh"

namespace osmos {
namespace ring {
namespace {

using namespace tma;
using staged::build_luts;
using staged::Rep;
using staged::RepLuts;
using staged::RepLuts2;
using staged::build_luts2;
using staged::Super;
using lanes::LaneAt;
using lanes::iq1m_block_sums;
using lanes::iq3_block_sums;
using lanes::sub_codes;

constexpr int kWarps = 16, kThreads = kWarps * kWarp;
constexpr int kMaxSlots = 4;
constexpr uint32_t kTaskRows = 32;  // rows a fused task has at most, a lane each (its tokens' loads are shared by them)
constexpr uint32_t kMaxEntries = 1024;  // entries a launch takes (their pointers and live list sit in shared memory)
constexpr uint32_t kSmemLimit = 226u * 1024u;

__device__ uint32_t g_status;

struct Args {
  const uint8_t* const* wg;
  const uint8_t* const* wu;
  const int32_t *cnt, *xrow, *xin, *win;
  const int8_t* q;
  const float* d;
  const float* scale;
  float lim;
  float* out;
  uint32_t rows, cols, out_stride, n_entries, max_cnt;
  uint32_t slots, slot_rows, task_slots, slot_bytes;  // a slot: slot_rows rows (of each matrix); a task: task_slots slots
  uint32_t list_off, ptr_off, ring_off;               // byte offsets into dynamic shared memory
  uint32_t* status;
  LaneEp ep;
};

// L: lanes a row; NB: blocks a lane holds at most (EXACT: exactly - no test a block, so the blocks' loads can be
// scheduled together); NT: tokens a task carries
template <uint32_t T, bool FUSED, int L, int NB, int NT, bool EXACT>
__global__ void __launch_bounds__(kThreads, 1) lane_ring_kernel(const Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[kWarps][kMaxSlots];
  __shared__ int s_scan[kWarps];
  __shared__ int s_pairs;
  constexpr int M = FUSED ? 2 : 1;
  constexpr int SB = Super<T>::bytes;
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t sub = lane % L, grp = lane / L;
  const uint32_t nblk = a.cols / 32, row_bytes = (a.cols / 256) * SB, nbl = nblk / L;
  const uint32_t S = a.slots, RC = a.slot_rows;
  uint16_t* list = (uint16_t*) (smem + a.list_off);
  const uint8_t** wptr = (const uint8_t**) (smem + a.ptr_off);
  int2* meta = (int2*) (wptr + a.n_entries * (FUSED ? 2 : 1));  // an entry's (live tokens, first row): no trip to the tables a task
  uint8_t* ring = smem + a.ring_off + warp * S * a.slot_bytes;

  if (lane == 0) {
    for (uint32_t s = 0; s < S; s++) bar_init(&full[warp][s], 1);
    bar_init_fence();
  }
  const RepLuts2<T> luts = build_luts2<T>(smem, kThreads);
  // (a dependent launch: the tables and activations read from here on may be the output of the kernels ahead; the
  // codebooks above are not)
  pdl_wait();
  pdl_launch_next();
  // (the expert-parallel step: the activations and weights of an odd step lie in the buffers' second halves)
  // (one register: the addresses are formed where a task loads its tokens, once a task)
  const uint32_t parity = a.ep.step ? (*a.ep.step & 1u) : 0u;
  auto out_row_ptr = [&](uint32_t r) -> float* {
    return a.ep.out_rows ? a.ep.out_rows[r] : a.out + (uint64_t) r * a.out_stride;
  };

  // the live (entry, token group) list in entry order, and every entry's matrix pointers
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
        mine = (c + NT - 1) / NT;
        const uint8_t* g = a.wg[m];
        wptr[m * M] = g;
        if (mine && ((uintptr_t) g & 15u)) aligned = false;
        if constexpr (FUSED) {
          const uint8_t* u = a.wu[m];
          wptr[m * M + 1] = u;
          if (mine && ((uintptr_t) u & 15u)) aligned = false;
        }
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
  // a matrix that is not 16-byte aligned cannot be copied in bulk: the whole launch stands down (nothing written)
  const int any_bad = __syncthreads_or(aligned ? 0 : 1);
  if (any_bad) {
    if (tid == 0) atomicOr(a.status, 2u);
    return;
  }
  // a task: at most a.task_slots slots, halved while the launch has fewer than four tasks a warp (few entries, as a
  // rank of many has: finer tasks fill the last round of warps better than they cost in activation loads)
  const uint32_t stride = gridDim.x * kWarps;
  uint32_t TS = a.task_slots;
  while (TS > 1 && (uint32_t) s_pairs * (a.rows / (RC * TS)) < 4u * stride) TS >>= 1;
  const uint32_t tpp = a.rows / (RC * TS);  // tasks an (entry, token group)
  const uint32_t tasks = (uint32_t) s_pairs * tpp;
  // this warp's place in the deal: neighbouring tasks go to different blocks, so every block gets the same share
  const uint32_t gw = warp * gridDim.x + blockIdx.x;

  // slot q of this warp's sequence: slot q % TS of its task q / TS
  auto issue = [&](uint32_t q) {  // one lane
    const uint32_t tk = gw + (q / TS) * stride;
    if (tk >= tasks) return;
    const uint32_t pair = tk / tpp, row0 = (tk - pair * tpp) * RC * TS + (q % TS) * RC;
    const uint32_t m = list[pair] & 0x3FFu, slot = q % S, bytes = RC * row_bytes;
    uint8_t* dst = ring + slot * a.slot_bytes;
    bar_expect(&full[warp][slot], M * bytes);
    bulk_load(dst, wptr[m * M] + (uint64_t) row0 * row_bytes, bytes, &full[warp][slot]);
    if constexpr (FUSED) bulk_load(dst + bytes, wptr[m * M + 1] + (uint64_t) row0 * row_bytes, bytes, &full[warp][slot]);
  };
  if (lane == 0)
    for (uint32_t q = 0; q < S; q++) issue(q);

  // the lane's blocks: block sub + L k is sub-block jj[k] of the superblock sboff[k] bytes into a row
  uint32_t sboff[NB];
#pragma unroll
  for (int k = 0; k < NB; k++) sboff[k] = ((sub + (uint32_t) L * k) >> 3) * SB;
  // (a row is a multiple of 4 bytes and the lane's superblocks lie an even count apart: one alignment for all)
  const uint32_t par = (SB % 4) ? ((sub >> 3) & 1u) * 2u : 0u;
  const LaneAt at{sub & 7u, 8u * (sub & 7u) + par, 16u - 8u * par};

  // one row's chain: the lane's blocks in order
  auto row_chain = [&](auto live_tag, uint32_t ra, const int (&xq)[NT][NB][8], const float (&xd)[NT][NB], float* acc) {
    constexpr int NTL = decltype(live_tag)::value;
#pragma unroll
    for (int k = 0; k < NB; k++) {
      if (EXACT || (uint32_t) k < nbl) {
        if constexpr (T == QTYPE_IQ3_XXS || T == QTYPE_IQ1_M) {
          float bs[NTL];
          if constexpr (T == QTYPE_IQ3_XXS) iq3_block_sums<NTL, NT, NB>(ra + sboff[k], at, luts, xq, k, bs);
          else iq1m_block_sums<NTL, NT, NB>(ra + sboff[k], at, luts, xq, k, bs);
#pragma unroll
          for (int t = 0; t < NTL; t++) acc[t] = __fmaf_rn(xd[t][k], bs[t], acc[t]);
        } else {
          LaneCodes c;
          sub_codes<T>(ra + sboff[k], at, c, luts);
#pragma unroll
          for (int t = 0; t < NTL; t++) acc[t] = __fmaf_rn(xd[t][k], lane_block_sum<T>(c, xq[t][k]), acc[t]);
        }
      }
    }
  };
  auto tree = [&](float v) -> float {
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, o, kWarp));
    return v;
  };

  // a slot's rows, for NTL live tokens
  // fused: a row's gate and up sums are kept by the lane whose index is the row's place in the task (hg, hu); the
  // task's rows get their activation together at its end, a lane a row
  auto do_slot = [&](auto live_tag, uint32_t sa, uint32_t row0, uint32_t place0, float* const (&orow)[NT],
                     const int (&xq)[NT][NB][8], const float (&xd)[NT][NB], float* hg, float* hu) {
    constexpr int NTL = decltype(live_tag)::value;
    const uint32_t half_bytes = RC * row_bytes;  // fused: the up rows follow the gate rows
    if constexpr (FUSED && L == 16) {
      for (uint32_t p = 0; p < RC; p++) {  // lanes 0 .. 15 the gate row, 16 .. 31 the up row
        float acc[NTL];
#pragma unroll
        for (int t = 0; t < NTL; t++) acc[t] = 0.0f;
        row_chain(live_tag, sa + grp * half_bytes + p * row_bytes, xq, xd, acc);
#pragma unroll
        for (int t = 0; t < NTL; t++) {
          const float v = tree(acc[t]);  // (lanes 0 .. 15: the gate row's sum, 16 .. 31: the up row's)
          const float gate = __shfl_sync(0xFFFFFFFFu, v, 0, kWarp), up = __shfl_sync(0xFFFFFFFFu, v, 16, kWarp);
          if (lane == place0 + p) hg[t] = gate, hu[t] = up;
        }
      }
    } else if constexpr (FUSED) {
      for (uint32_t p = 0; p < RC; p++) {  // the whole warp the gate row, then the up row
        float ag[NTL], au[NTL];
#pragma unroll
        for (int t = 0; t < NTL; t++) ag[t] = 0.0f, au[t] = 0.0f;
        row_chain(live_tag, sa + p * row_bytes, xq, xd, ag);
        row_chain(live_tag, sa + half_bytes + p * row_bytes, xq, xd, au);
#pragma unroll
        for (int t = 0; t < NTL; t++) {
          const float g = tree(ag[t]), u = tree(au[t]);
          if (lane == place0 + p) hg[t] = g, hu[t] = u;
        }
      }
    } else {
      constexpr uint32_t RU = kWarp / L;  // rows at once
      for (uint32_t p = 0; p < RC; p += RU) {
        float acc[NTL];
#pragma unroll
        for (int t = 0; t < NTL; t++) acc[t] = 0.0f;
        row_chain(live_tag, sa + (p + grp) * row_bytes, xq, xd, acc);
#pragma unroll
        for (int t = 0; t < NTL; t++) {
          const float v = tree(acc[t]);
          if (sub == 0) orow[t][row0 + p + grp] = v;
        }
      }
    }
  };

  using I1 = std::integral_constant<int, 1>;
  using I2 = std::integral_constant<int, NT>;
  for (uint32_t n = 0;; n++) {
    const uint32_t tk = gw + n * stride;
    if (tk >= tasks) break;
    const uint32_t pair = tk / tpp, task_row0 = (tk - pair * tpp) * RC * TS;
    const uint32_t v = list[pair], m = v & 0x3FFu, g = v >> 10;
    const int2 me = meta[m];
    const uint32_t cnt = (uint32_t) me.x, live = cnt - g * NT < (uint32_t) NT ? cnt - g * NT : (uint32_t) NT;
    const uint32_t r0 = (uint32_t) me.y + g * NT;
    // the task's tokens: the lane's blocks of their int8 rows, their scales, the routed weights
    int xq[NT][NB][8];
    float xd[NT][NB], scale[NT];
    float* orow[NT];  // where each token's results go: looked up now, used when the task's rows are done
    const int8_t* const in_q = a.q + parity * a.ep.half_q;
    const float* const in_d = (const float*) ((const uint8_t*) a.d + parity * a.ep.half_d);
#pragma unroll
    for (int t = 0; t < NT; t++) {
      const uint32_t r = r0 + ((uint32_t) t < live ? (uint32_t) t : live - 1);
      const uint64_t xr = a.xin ? (uint64_t) (uint32_t) a.xin[r] : r;
      orow[t] = out_row_ptr(r);
      scale[t] = 0.0f;
      if constexpr (FUSED) scale[t] = ((const float*) ((const uint8_t*) a.scale + parity * a.ep.half_scale))[a.win ? a.win[r] : r];
#pragma unroll
      for (int k = 0; k < NB; k++) {
        int4 lo = make_int4(0, 0, 0, 0), hi = lo;
        float dv = 0.0f;
        if (EXACT || (uint32_t) k < nbl) {
          const uint32_t s = sub + (uint32_t) L * k;
          const int4* xp = (const int4*) (in_q + xr * a.cols + s * 32u);
          lo = __ldg(xp), hi = __ldg(xp + 1), dv = __ldg(in_d + xr * nblk + s);
        }
        xq[t][k][0] = lo.x, xq[t][k][1] = lo.y, xq[t][k][2] = lo.z, xq[t][k][3] = lo.w;
        xq[t][k][4] = hi.x, xq[t][k][5] = hi.y, xq[t][k][6] = hi.z, xq[t][k][7] = hi.w;
        xd[t][k] = dv;
      }
    }
    float hg[NT], hu[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) hg[t] = 0.0f, hu[t] = 0.0f;
    bool ok = true;
    for (uint32_t ss = 0; ss < TS; ss++) {
      const uint32_t q = n * TS + ss, slot = q % S;
      if (!bar_wait(&full[warp][slot], (q / S) & 1u)) {  // a copy never landed: report it and leave
        ok = false;
        break;
      }
      const uint32_t sa = smem_addr(ring + slot * a.slot_bytes);
      if (NT > 1 && live == (uint32_t) NT) do_slot(I2{}, sa, task_row0 + ss * RC, ss * RC, orow, xq, xd, hg, hu);
      else do_slot(I1{}, sa, task_row0 + ss * RC, ss * RC, orow, xq, xd, hg, hu);
      __syncwarp();  // every lane is done reading the slot: refill it
      if (lane == 0) {
        fence_async_smem();
        issue(q + S);
      }
    }
    if (!ok) {
      if (lane == 0) atomicOr(a.status, 1u);
      break;
    }
    if constexpr (FUSED) {
      if (lane < RC * TS) {
#pragma unroll
        for (int t = 0; t < NT; t++)
          if ((uint32_t) t < live)
            orow[t][task_row0 + lane] = lane_swiglu(hg[t], hu[t], a.lim, scale[t]);
      }
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

template <uint32_t T, bool FUSED, int L, int NB, int NT, bool EXACT>
int launch(const Request& r, cudaStream_t s) {
  const Device* dev = device_info();
  if (!dev) return 0;
  constexpr uint32_t M = FUSED ? 2 : 1, RU = FUSED ? 1 : kWarp / L;
  const uint32_t row_bytes = r.cols / 256 * Super<T>::bytes;
  Args a{};
  a.list_off = (uint32_t) ((Rep<T>::bytes + 127) & ~127);
  a.ptr_off = a.list_off + kMaxEntries * (8 / NT) * 2;
  a.ring_off = (a.ptr_off + r.n_entries * (M * 8 + 8) + 127u) & ~127u;  // (pointers, then (count, first row))
  if (a.ring_off + 16u >= kSmemLimit) return 0;
  // a slot: the fewest rows (a multiple of the rows a pass takes) whose bytes are a multiple of 16 and reach about 3 KB
  uint32_t rc = RU;
  while ((rc * row_bytes) % 16u) rc += RU;
  while (M * rc * row_bytes < 3072u && r.rows % (2 * rc) == 0) rc *= 2;
  if (r.rows % rc) return 0;
  if (FUSED && rc > 32) return 0;  // (a fused task's rows each have a lane)
  const uint32_t slot_bytes = M * rc * row_bytes;
  uint32_t slots = (kSmemLimit - a.ring_off - 16u) / (kWarps * slot_bytes);
  if (slots > (uint32_t) kMaxSlots) slots = kMaxSlots;
  if (slots < 2) return 0;
  // a task: slots of one entry that share the activation registers - about 8 rows of work a token's loads
  uint32_t ts = 1;
  while (ts * rc < (FUSED ? kTaskRows : 8u) && r.rows % (2 * ts * rc) == 0) ts *= 2;
  if (FUSED && ts * rc > 32) return 0;
  a.wg = (const uint8_t* const*) r.wg, a.wu = (const uint8_t* const*) r.wu, a.cnt = r.cnt, a.xrow = r.xrow, a.xin = r.xin;
  a.win = r.win, a.q = r.q, a.d = r.d, a.scale = r.scale, a.lim = r.lim, a.out = r.out, a.rows = r.rows, a.cols = r.cols;
  a.out_stride = r.out_stride, a.n_entries = r.n_entries, a.max_cnt = r.max_cnt;
  a.slots = slots, a.slot_rows = rc, a.task_slots = ts, a.slot_bytes = slot_bytes;
  a.status = dev->status;
  a.ep = r.ep;
  const uint32_t total = a.ring_off + kWarps * slots * slot_bytes + 16u;
  if (r.dry) return 1;
  static bool sized[64] = {};  // (per template instance and device: the attribute belongs to a device's context)
  auto kernel = lane_ring_kernel<T, FUSED, L, NB, NT, EXACT>;
  if (!allow_dynamic_smem(kernel, (int) kSmemLimit, sized)) return 0;
  return launch_dependent(kernel, dim3((uint32_t) dev->sms), dim3(kThreads), total, s, a) == cudaSuccess ? 1 : -1;
}

template <uint32_t T, bool FUSED>
int by_shape(const Request& r, cudaStream_t s) {
  const uint32_t nblk = r.cols / 32;
  if (r.cols < 4096) {
    if (nblk % 16) return 0;
    const uint32_t per = nblk / 16;
    if (per == 1) return launch<T, FUSED, 16, 1, 2, true>(r, s);
    if (per == 4) return launch<T, FUSED, 16, 4, 2, true>(r, s);
    if (per < 4) return launch<T, FUSED, 16, 4, 2, false>(r, s);
    return 0;
  }
  if (nblk % 32) return 0;
  const uint32_t per = nblk / 32;
  if (per == 4) return launch<T, FUSED, 32, 4, 2, true>(r, s);
  if (per < 4) return launch<T, FUSED, 32, 4, 2, false>(r, s);
  if (per <= 8) return launch<T, FUSED, 32, 8, 1, false>(r, s);
  return 0;
}

}  // namespace

int try_launch(uint32_t type, const Request& r, void* stream) {
  if (r.cols % 256 || !r.rows || !r.n_entries || r.n_entries > kMaxEntries || !r.max_cnt || r.max_cnt > 8) return 0;
  if (((uintptr_t) r.q & 15u) || ((uintptr_t) r.d & 3u)) return 0;
  const cudaStream_t s = (cudaStream_t) stream;
#define CASE(T)                                    \
  if (r.fused) return by_shape<T, true>(r, s);     \
  return by_shape<T, false>(r, s);
  switch (type) {
    case QTYPE_IQ3_XXS: CASE(QTYPE_IQ3_XXS)
    case QTYPE_IQ1_M: CASE(QTYPE_IQ1_M)
    case QTYPE_IQ2_XXS: CASE(QTYPE_IQ2_XXS)
    case QTYPE_IQ1_S: CASE(QTYPE_IQ1_S)
    default: return 0;
  }
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

}  // namespace ring
}  // namespace osmos
