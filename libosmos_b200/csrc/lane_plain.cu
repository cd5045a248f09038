// q8_run for the plain 32-value blocks (Q4_0, Q8_0), one or two tokens: the int8 lane's sums
//   block = d_w (float) sum_i w_i x_i (exact integer),  acc = fmaf(d_x[block], block, acc),
// blocks dealt to L = 16 lanes (32 from 4096 columns), lane l taking blocks l, l + L, ... in order, then the xor tree
// over the L lanes - the order q8.cu's generic kernel gives these types.
//
// Every lane keeps the int8 x of its blocks (and their scales, and for Q4_0 their sums) in registers for the whole
// launch; the weights come through shared memory by bulk copies, each warp owning a ring of slots it fills and drains
// by itself (no block-wide barrier after the start). Q4_0's nibbles are used as they lie, unsigned: sum (n - 8) x =
// sum n x - 8 sum x, the second sum worked out once a launch. That leaves about one instruction a weight value, so
// the kernel waits on memory, not on its arithmetic.
#include "lane_plain_api.h"

#include "decode.cuh"
#include "tma.cuh"

namespace osmos {
namespace plain {
namespace {

using namespace tma;

constexpr int kMaxSlots = 4;
constexpr uint32_t kSmemLimit = 224u * 1024u;

__device__ uint32_t g_status;

struct Args {
  const uint8_t* w;
  const int8_t* q;
  const float* d;
  float* y;
  uint32_t rows, cols, ys, n_tok;
  uint32_t slots, slot_rows, slot_bytes, units;  // a unit: the rows of one slot
  uint32_t* status;
};

template <uint32_t T> struct Plain;
template <> struct Plain<QTYPE_Q4_0> { static constexpr int bytes = 18, words = 4; };
template <> struct Plain<QTYPE_Q8_0> { static constexpr int bytes = 34, words = 8; };

__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {  // unsigned bytes of a x signed bytes of b
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// L: lanes a row; NB: blocks a lane holds (a power of two, cols <= 32 L NB); NT: tokens; W: warps a block
template <uint32_t T, int L, int NB, int NT, int W>
__global__ void __launch_bounds__(W * kWarp, (W <= 12 ? 2 : 1)) plain_dense_kernel(const Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[W][kMaxSlots];
  constexpr int RU = kWarp / L;  // rows a warp sums at once
  constexpr int NQ = Plain<T>::words;
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t sub = lane % L, grp = lane / L;
  const uint32_t nblk = a.cols / 32, row_bytes = nblk * Plain<T>::bytes;
  const uint32_t S = a.slots;
  uint8_t* ring = smem + warp * S * a.slot_bytes;

  const uint32_t u_lo = (uint32_t) ((uint64_t) blockIdx.x * a.units / gridDim.x);
  const uint32_t u_hi = (uint32_t) ((uint64_t) (blockIdx.x + 1) * a.units / gridDim.x);
  auto issue = [&](uint32_t i) {  // one lane: the warp's i-th unit into slot i % S
    const uint32_t u = u_lo + warp + i * W;
    if (u >= u_hi) return;
    const uint32_t r0 = u * a.slot_rows, nrows = a.rows - r0 < a.slot_rows ? a.rows - r0 : a.slot_rows;
    const uint32_t slot = i % S, bytes = nrows * row_bytes;
    bar_expect(&full[warp][slot], bytes);
    bulk_load(ring + slot * a.slot_bytes, a.w + (uint64_t) r0 * row_bytes, bytes, &full[warp][slot]);
  };
  if (lane == 0) {
    for (uint32_t s = 0; s < S; s++) bar_init(&full[warp][s], 1);
    bar_init_fence();
    for (uint32_t i = 0; i < S; i++) issue(i);
  }
  // Launched as a programmatic dependent of the kernel before it on the stream: this block may have started while
  // that kernel was still finishing, and what ran so far touched only the weights (which no kernel writes). The
  // activations may be that kernel's output: wait for it here. The kernel after this one may start the same way.
  pdl_wait();
  pdl_launch_next();

  // The lane's blocks are sub, sub + L, ...; it reads them in the order p -> block sub + L ((p + rot) % NB), where
  // the second row's lanes start half-way round: rows are a multiple of 128 bytes apart, so without the turn both
  // rows' lanes would ask the same shared-memory banks at once. Position p's x is kept at index p.
  const uint32_t rot = grp * (NB / 2);
  int xq[NT][NB][8];
  float xd[NT][NB];
  int xsum[NT][NB];
  uint32_t boff[NB];  // position p's block: its byte offset in a row (a block past the row reads the last one's bytes)
  bool live[NB];
#pragma unroll
  for (int p = 0; p < NB; p++) {
    const uint32_t s = sub + (uint32_t) L * ((p + rot) % NB);
    live[p] = s < nblk;
    boff[p] = (live[p] ? s : nblk - 2 + (sub & 1u)) * Plain<T>::bytes;  // (of the lane's own parity)
#pragma unroll
    for (int t = 0; t < NT; t++) {
      const uint32_t tt = (uint32_t) t < a.n_tok ? (uint32_t) t : a.n_tok - 1;  // a slot past the tokens repeats the last
      int4 lo = make_int4(0, 0, 0, 0), hi = lo;
      float dv = 0.0f;
      if (live[p]) {
        const int4* xp = (const int4*) (a.q + (uint64_t) tt * a.cols + s * 32u);
        lo = __ldg(xp), hi = __ldg(xp + 1), dv = __ldg(a.d + (uint64_t) tt * nblk + s);
      }
      xq[t][p][0] = lo.x, xq[t][p][1] = lo.y, xq[t][p][2] = lo.z, xq[t][p][3] = lo.w;
      xq[t][p][4] = hi.x, xq[t][p][5] = hi.y, xq[t][p][6] = hi.z, xq[t][p][7] = hi.w;
      xd[t][p] = dv;
      int sx = 0;
#pragma unroll
      for (int j = 0; j < 8; j++) sx = __dp4a(0x01010101, xq[t][p][j], sx);
      xsum[t][p] = 8 * sx;
    }
  }
  __syncthreads();  // the barriers' initialisation, seen by every lane that will wait on them

  // where a block's bytes lie in the words around it: a row starts on a 16-byte boundary and a block is 2 mod 4
  // bytes long, so block s starts 0 (s even) or 2 (s odd) bytes into a word - and s's parity is the lane's
  const uint32_t odd = sub & 1u;
  const uint32_t qsh = odd ? 32u : 16u;  // the codes start 2 bytes after the block: the next word (odd) or mid-word
  const uint32_t dsh = odd ? 16u : 0u;   // the f16 scale: the word's high (odd) or low half

  for (uint32_t i = 0;; i++) {
    const uint32_t u = u_lo + warp + i * W;
    if (u >= u_hi) break;
    const uint32_t slot = i % S;
    if (!bar_wait(&full[warp][slot], (i / S) & 1u)) {  // a copy never landed: report it and leave
      if (lane == 0) atomicOr(a.status, 1u);
      break;
    }
    const uint32_t sa = smem_addr(ring + slot * a.slot_bytes);
    const uint32_t r0 = u * a.slot_rows;
    for (uint32_t rr = 0; rr < a.slot_rows; rr += RU) {
      const uint32_t row = r0 + rr + grp;  // (a row past the matrix: summed from stale bytes, never stored)
      const uint32_t ra = sa + (rr + grp) * row_bytes;
      uint32_t wv[NB][NQ + 1];
#pragma unroll
      for (int p = 0; p < NB; p++) {
        const uint32_t al = (ra + boff[p]) & ~3u;
#pragma unroll
        for (int j = 0; j <= NQ; j++) wv[p][j] = lds32(al + 4 * j);
      }
      float bs[NT][NB];  // position p's block sum
#pragma unroll
      for (int p = 0; p < NB; p++) {
        const float dw = half_value((wv[p][0] >> dsh) & 0xFFFFu);
        uint32_t c[NQ];
#pragma unroll
        for (int j = 0; j < NQ; j++) c[j] = __funnelshift_rc(wv[p][j], wv[p][j + 1], qsh);
#pragma unroll
        for (int t = 0; t < NT; t++) {
          int isum = 0;
          if constexpr (T == QTYPE_Q4_0) {
            // the nibbles as they lie: the high ones stay in place, their dot 16 times too large (exactly)
            int hi16 = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              isum = __dp4a((int) (c[j] & 0x0F0F0F0Fu), xq[t][p][j], isum);
              hi16 = dp4a_us(c[j] & 0xF0F0F0F0u, xq[t][p][4 + j], hi16);
            }
            isum += (hi16 >> 4) - xsum[t][p];
          } else {
#pragma unroll
            for (int j = 0; j < 8; j++) isum = __dp4a((int) c[j], xq[t][p][j], isum);
          }
          bs[t][p] = mul_rn(dw, (float) isum);
        }
      }
#pragma unroll
      for (int t = 0; t < NT; t++) {
        float acc = 0.0f;
#pragma unroll
        for (int ib = 0; ib < NB; ib++) {  // the lane's blocks in order: block ib sits at position (ib - rot) % NB
          const int p0 = ib, p1 = (ib + NB - NB / 2) % NB;
          const float b = grp ? bs[t][p1] : bs[t][p0], dxv = grp ? xd[t][p1] : xd[t][p0];
          const bool on = grp ? live[p1] : live[p0];
          const float next = __fmaf_rn(dxv, b, acc);
          acc = on ? next : acc;
        }
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, o, kWarp));
        if (sub == 0 && row < a.rows && (uint32_t) t < a.n_tok) a.y[(uint64_t) t * a.ys + row] = acc;
      }
    }
    __syncwarp();  // every lane is done reading the slot: refill it
    if (lane == 0) {
      fence_async_smem();
      issue(i + S);
    }
  }
}

struct Device {
  int sms = 0;
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
    devs[d].sms = sms, devs[d].status = (uint32_t*) at;
  }
  return &devs[d];
}

template <uint32_t T, int L, int NB, int NT, int W>
int launch(const Request& r, cudaStream_t s) {
  const Device* dev = device_info();
  if (!dev) return 0;
  constexpr uint32_t RU = kWarp / L;
  const uint32_t row_bytes = r.cols / 32 * Plain<T>::bytes;
  // a slot's rows: as many (1, 2 or 4 passes of the warp) as leave every warp two slots' worth of rows and the ring
  // three slots; a small matrix takes one pass a slot so that its rows spread over every warp of every block
  uint32_t slot_rows = RU, slots = 0;
  for (uint32_t k = 4; k >= 1; k >>= 1) {
    const uint32_t rows_k = RU * k, n = kSmemLimit / (W * rows_k * row_bytes);
    if (k > 1 && (n < 3 || (uint64_t) r.rows < 2ull * rows_k * W * dev->sms)) continue;
    slot_rows = rows_k, slots = n > (uint32_t) kMaxSlots ? (uint32_t) kMaxSlots : n;
    break;
  }
  if (slots < 1) return 0;
  Args a{};
  a.w = (const uint8_t*) r.w, a.q = r.q, a.d = r.d, a.y = r.y, a.rows = r.rows, a.cols = r.cols, a.ys = r.ys;
  a.n_tok = r.n_tok, a.slots = slots, a.slot_rows = slot_rows, a.slot_bytes = slot_rows * row_bytes;
  a.units = (r.rows + slot_rows - 1) / slot_rows;
  a.status = dev->status;
  {
    // no more slots than a warp has units: a small matrix then leaves shared memory for the next launch's blocks,
    // which start their weight copies beside this launch's (a programmatic dependent waits only for its activations)
    const uint32_t blocks = a.units < (uint32_t) dev->sms ? a.units : (uint32_t) dev->sms;
    const uint32_t per_warp = ((a.units + blocks - 1) / blocks + W - 1) / W;
    if (per_warp < slots) slots = per_warp, a.slots = per_warp;
  }
  const uint32_t total = W * slots * a.slot_bytes + 16u;  // + the word read past a last block
  static bool sized[64] = {};  // (one record a template instance, one flag a device)
  auto kernel = plain_dense_kernel<T, L, NB, NT, W>;
  if (!allow_dynamic_smem(kernel, (int) kSmemLimit + 16, sized)) return 0;
  uint32_t grid = (uint32_t) dev->sms;
  if (a.units < grid) grid = a.units;
  return launch_dependent(kernel, dim3(grid), dim3(W * kWarp), total, s, a) == cudaSuccess ? 1 : -1;
}

// blocks a lane: the power of two that holds cols / 32 / L
template <uint32_t T, int L, int NT>
int by_blocks(const Request& r, cudaStream_t s) {
  const uint32_t per = (r.cols / 32 + L - 1) / L;
  if constexpr (NT == 1) {
    // a matrix of at most two passes a warp of the small block: twelve warps, two blocks a multiprocessor, so that the
    // launch behind this one is resident (its copies in flight) while this one computes
    const Device* dev = device_info();
    if (dev && (uint64_t) r.rows <= 2ull * (kWarp / L) * 12u * (uint32_t) dev->sms) {
      if (per <= 1) return launch<T, L, 1, 1, 12>(r, s);
      if (per <= 2) return launch<T, L, 2, 1, 12>(r, s);
      if (per <= 4) return launch<T, L, 4, 1, 12>(r, s);
    }
  }
  if (per <= 1) return launch<T, L, 1, NT, (NT == 1 ? 24 : 16)>(r, s);
  if (per <= 2) return launch<T, L, 2, NT, (NT == 1 ? 24 : 16)>(r, s);
  if (per <= 4) return launch<T, L, 4, NT, (NT == 1 ? 24 : 16)>(r, s);
  if constexpr (NT == 1)
    if (per <= 8) return launch<T, L, 8, 1, 16>(r, s);
  return 0;
}

template <uint32_t T>
int by_shape(const Request& r, cudaStream_t s) {
  if (r.cols % 256 || r.n_tok > 2) return 0;  // a row's bytes are then a multiple of 16: a bulk copy's
  if (r.cols < 4096) return r.n_tok == 1 ? by_blocks<T, 16, 1>(r, s) : by_blocks<T, 16, 2>(r, s);
  return r.n_tok == 1 ? by_blocks<T, 32, 1>(r, s) : by_blocks<T, 32, 2>(r, s);
}

}  // namespace

int try_launch(uint32_t type, const Request& r, void* stream) {
  if (!r.rows || !r.n_tok) return 0;
  if (((uintptr_t) r.w | (uintptr_t) r.q) & 15u || (uintptr_t) r.d & 3u) return 0;
  if (r.n_tok > 1 && r.cols % 16) return 0;
  if (type == QTYPE_Q4_0) return by_shape<QTYPE_Q4_0>(r, (cudaStream_t) stream);
  if (type == QTYPE_Q8_0) return by_shape<QTYPE_Q8_0>(r, (cudaStream_t) stream);
  return 0;
}

uint32_t read_status() {
  const Device* dev = device_info();
  if (!dev) return 0x80000000u;
  uint32_t v = 0, zero = 0;
  if (cudaMemcpy(&v, dev->status, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return 0x80000000u;
  cudaMemcpy(dev->status, &zero, sizeof zero, cudaMemcpyHostToDevice);
  return v;
}

}  // namespace plain
}  // namespace osmos
