// FP4 weights times FP4 activations on the 5th-generation tensor cores: tcgen05.mma with block scales, both operands'
// scale factors in tensor memory (fp4_tc_api.h). Two forms of one kernel:
//   NVFP4 (kind::mxf4nvf4, a UE4M3 scale every 16 values): ggml type 40 weights against mm_fp4_act's activations - the
//         product the reference runs on sm_120a's mma.sync kind::mxf4nvf4 (kernels/mm_fp4.hip:149-259);
//   MXFP4 (kind::mxf4, a UE8M0 scale every 32 values): ggml type 39 weights against ops_fp4_round's packed activations.
// E2M1 x E2M1 products are exact and so is a product of two scale factors; the sums are the tensor core's, in F32.
//
// A block computes 128 weight rows x up to 256 tokens; K in steps of 256 values through a ring of four stages.
//   producers (8 warps)  the rows' blocks as the GGUF holds them -> the tensor core's operand layout: the nibbles
//                        reordered from ggml's "low nibbles first, then high" to K order (two values a byte, the lower K
//                        in the low nibble) into K-major core matrices of 8 rows x 16 bytes, and the block scales into
//                        the scale-factor chunk layout (128 rows x 4 factors: byte (r % 32) * 16 + (r / 32) * 4 + f).
//                        The raw bytes reach shared memory by the loader's tensor-map copies (a ring of its own, three
//                        stages ahead), so a producer only ever waits on shared memory. The tokens' scale bytes go to
//                        the chunk layout by 4-byte cp.async that nobody waits for (the stage's barrier counts them).
//   loaders (2 warps)    one the rows' raw bytes (a box of 128 rows x 144 bytes a stage), one the tokens' codes, already in
//                        K order: one tensor-map copy a stage, a box of 256 tokens x 128 bytes written with the 128-byte
//                        swizzle, which the MMA's B descriptor names (an MMA's 32 bytes of K 32 bytes along the row).
//   issuer (1 warp)      per 64 values of K: tcgen05.cp of the scale-factor chunks into tensor memory (32 lanes x 16
//                        bytes, broadcast to the four lane quarters), then one tcgen05.mma M128 N(16 .. 256) K64 with
//                        the chunks' addresses; tcgen05.commit onto the stage's "empty" barrier after a stage's four,
//                        onto the accumulator's barrier after the last.
//   epilogue (4 warps)   thread = one weight row (its TMEM lane): tcgen05.ld the sums, times the tensors' scale, stored.
// The descriptors follow the layouts CUTLASS documents in cute/arch/mma_sm100_desc.hpp (InstrDescriptorBlockScaled),
// cute/atom/mma_traits_sm100.hpp (the scale factors' tensor-memory fragment) and cutlass/detail/sm100_blockscaled_layout.hpp
// (the chunk layout); tests/test_fp4_desc.py holds the instruction descriptor to CUTLASS's own encoder.
//
// Every mbarrier wait is bounded (%globaltimer); a wait that runs out raises the status word, every role falls through
// to the common exit and tensor memory is released.
#include "fp4_tc_api.h"

#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace osmos {
namespace fp4_tc {
namespace {

constexpr int kM = 128, kNMax = 256;
constexpr int kEpiWarps = 4, kProdWarps = 8;
// Who does what goes by the warp scheduler a warp lives on (its index mod 4). Scheduler 0 has the issuer and the two
// loaders, which issue little and wait much, and an epilogue warp that sleeps until the end - so the issuer, whose
// chain of tcgen05 instructions a stage is the kernel's critical path (35 cycles a scale-factor copy, 75 an MMA, measured
// by leaving them out), never waits for an issue slot behind a producer. The eight producers share schedulers 1, 2 and 3
// with the other three epilogue warps. (A second issuing warp for the scale factors' copies, a stage ahead with two sets
// of tensor-memory columns, was slower: what the hand-over costs exceeds what the copies' issue saved.)
constexpr int kIssuerWarp = 4;   // scheduler 0
constexpr int kRawWarp = 8;      // scheduler 0: the rows' raw bytes by tensor-map copies
constexpr int kLoaderWarp = 12;  // scheduler 0: the tokens' codes by tensor-map copies
// producer p's warp: 5, 6, 7, 9, 10, 11, 13, 14
__host__ __device__ constexpr int producer_of(int warp) {  // 0 .. 7, or -1
  return (warp < 5 || warp > 14 || warp % 4 == 0) ? -1 : (warp / 4 - 1) * 3 + warp % 4 - 1;
}
static_assert(producer_of(5) == 0 && producer_of(7) == 2 && producer_of(9) == 3 && producer_of(11) == 5 && producer_of(13) == 6 &&
                  producer_of(14) == 7 && producer_of(8) == -1 && producer_of(12) == -1 && producer_of(4) == -1,
              "eight producers on schedulers 1 to 3");
constexpr int kProdThreads = kProdWarps * kWarp;
constexpr int kTasks = kM * 4 / kProdThreads;  // (row, MMA) tasks a producer thread takes a stage: 2
constexpr int kThreads = 15 * kWarp;
constexpr int kStages = 3, kRawStages = 3;
constexpr int kStepValues = 256, kMmaK = 64, kMmas = kStepValues / kMmaK;  // a stage: 256 values of K, four MMAs
constexpr int kABytes = kM * kStepValues / 2;                              // 16 KB: 128 rows of 128 bytes, the tokens' layout
constexpr int kBBytes = kNMax * kStepValues / 2;                           // 32 KB
constexpr int kChunk = 512;                                                // a scale-factor chunk: 128 rows x 4 factors
constexpr int kSfaBytes = 4 * kChunk, kSfbBytes = 2 * 4 * kChunk;          // at most 4 chunks of K a stage; B: two row halves
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;     // 54 KB
static_assert(kABytes % 1024 == 0 && kStageBytes % 1024 == 0, "both tiles start on 1024 bytes: the swizzle's period");
constexpr int kRawRow = 144;                // a row's raw bytes of one stage: 4 x 36 (NVFP4), or 8 x 17 = 136 and the 8 a
constexpr int kRawBytes = kM * kRawRow;     // 16-byte window may start before them (MXFP4)
constexpr uint64_t kWaitLimitNs = 200ull * 1000 * 1000;
// tensor memory: the accumulator's 256 columns, then the scale factors of one stage (a column = 4 factors of 32 rows)
constexpr uint32_t kSfaCol = 256, kSfbCol = kSfaCol + 16, kTmemCols = 512;

__device__ uint32_t g_status;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = smem_addr(bar);
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; spin++) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(a), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin == 0) t0 = global_ns();
    else if (global_ns() - t0 > kWaitLimitNs) return false;
  }
}

// shared-memory matrix descriptor: K-major, no swizzle, core matrices of 8 rows x 16 bytes; lbo: to the next 16 bytes of
// K, sbo: to the next 8 rows (cute/arch/mma_sm100_desc.hpp: start >> 4, leading >> 4 at bit 16, stride >> 4 at bit 32,
// version 1 at bit 46, layout type 0)
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) (lbo_bytes >> 4) << 16 | (uint64_t) (sbo_bytes >> 4) << 32 |
         (uint64_t) 1 << 46;
}

// the same for the tokens' tile as the tensor-map copy writes it with the 128-byte swizzle: rows of 128 bytes (a stage's K of
// a token), 8 rows 1024 bytes on; an MMA's 32 bytes of K start 32 bytes further into the row (layout type 2 at bit 61)
__device__ __forceinline__ uint64_t tile_desc_sw128(uint32_t addr) {
  return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) 1 << 16 | (uint64_t) (1024u >> 4) << 32 | (uint64_t) 1 << 46 | (uint64_t) 2 << 61;
}

// where the 16 bytes j (0 .. 7) of row r's 128 bytes of K lie in a tile under the 128-byte swizzle: rows of 128 bytes, a
// row's 16-byte pieces permuted by its place among its eight (what a tensor-map copy with that swizzle writes)
__device__ __forceinline__ uint32_t tile_at(uint32_t r, uint32_t j) { return r * 128u + ((j ^ (r & 7u)) << 4); }
// where row r's four factors lie in a scale-factor chunk (r < 128)
__device__ __forceinline__ uint32_t chunk_at(uint32_t r) { return (r & 31u) * 16u + (r >> 5) * 4u; }

// 16 values' nibbles to K order: `lo`, `hi` hold 8 bytes whose low nibbles are values 0 .. 7 and high nibbles values
// 8 .. 15 (ggml's order); returns values 0 .. 7 and 8 .. 15 as two words, value j at bits 4 (j % 8)
__device__ __forceinline__ uint2 k_order16(uint32_t lo, uint32_t hi) {
  const uint32_t m = 0x0F0F0F0Fu;
  const uint32_t a0 = lo & m, a1 = hi & m, b0 = (lo >> 4) & m, b1 = (hi >> 4) & m;
  // n | n' << 4 of neighbouring bytes lands in the even bytes; the two words' even bytes make one word
  return make_uint2(__byte_perm(a0 | a0 >> 4, a1 | a1 >> 4, 0x6420), __byte_perm(b0 | b0 >> 4, b1 | b1 >> 4, 0x6420));
}

struct Args {
  const uint8_t* w;        // the weight matrix, rows of GGUF blocks
  const uint8_t* aq;       // the tokens' codes, K order; a token's row aq_stride bytes on
  const uint8_t* as;       // the tokens' scale bytes; a token's row as_stride bytes on
  float* y;
  uint32_t rows, cols, n, ys, aq_stride, as_stride;
  float scale;
  uint32_t* status;
};

struct Shared {
  uint64_t full[kStages], empty[kStages], raw_full[kRawStages], raw_empty[kRawStages], acc_full;
  uint32_t tmem_base;
  int fail;
};

// MX false: NVFP4 (a 36-byte block of 64 values: 4 UE4M3 bytes, then 8 bytes a 16); MX true: MXFP4 (a 17-byte block of
// 32 values: the E8M0 byte, then 16 bytes)
template <bool MX>
__global__ void __launch_bounds__(kThreads, 1) fp4_tc_kernel(const Args a, const __grid_constant__ CUtensorMap tmap,
                                                             const __grid_constant__ CUtensorMap wmap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ Shared sh;
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t row0 = blockIdx.x * kM, c0 = blockIdx.y * kNMax;
  const uint32_t n_valid = a.n - c0 < (uint32_t) kNMax ? a.n - c0 : (uint32_t) kNMax;
  const uint32_t n_mma = (n_valid + 15u) & ~15u;  // the MMA's N: whole 16s
  const uint32_t steps = a.cols / kStepValues;
  constexpr uint32_t kSfChunks = MX ? 2 : 4;  // chunks of 4 factors a stage: 256 values / (4 x 32) or / (4 x 16)
  const uint64_t row_bytes = MX ? (uint64_t) (a.cols / 32) * 17 : (uint64_t) (a.cols / 64) * 36;

  if (tid == 0) {
    // a stage is full when every producer has stored its part of A (an arrival each), every producer's scale-byte copies
    // have landed (an arrival each, made by the copy engine) and the loader's tensor-map copy has delivered its bytes
    // (the producers arrive a warp at a time: an arrival is an atomic on shared memory, and hundreds a stage would be the
    // slowest thing in the kernel)
    for (int i = 0; i < kStages; i++) bar_init(&sh.full[i], kProdWarps + 1), bar_init(&sh.empty[i], 1);
    for (int i = 0; i < kRawStages; i++) bar_init(&sh.raw_full[i], 1), bar_init(&sh.raw_empty[i], kProdWarps);
    bar_init(&sh.acc_full, 1);
    sh.fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == (uint32_t) kIssuerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sh.tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sh.tmem_base;

  if (producer_of((int) warp) >= 0) {
    // ================= producers =================
    const uint32_t pt = (uint32_t) producer_of((int) warp) * kWarp + lane;
    const uint32_t raw0 = smem_addr(smem + kStages * kStageBytes);
    // this thread's token of the block: a warp takes tokens 8 b .. 8 b + 7 of each of a half's four 32-token groups,
    // whose words lie side by side in a chunk (32 lanes on 32 banks). A stage's scale bytes of a token are 16 (8)
    // bytes in a row: one load.
    const uint32_t sf_j = pt & 127u, sf_t128 = ((sf_j >> 3) & 3u) * 32u + (sf_j >> 5) * 8u + (sf_j & 7u);
    const uint32_t sf_t = (pt >> 7) * 128u + sf_t128, sf_at = chunk_at(sf_t128);
    const uint8_t* sf_row = a.as + (uint64_t) (c0 + (sf_t < n_valid ? sf_t : n_valid - 1)) * a.as_stride;
    uint32_t sfw[kSfChunks];
    auto read_sf = [&](uint32_t it) {
      if constexpr (MX)
        asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(sfw[0]), "=r"(sfw[1]) : "l"(sf_row + (uint64_t) it * 8u));
      else
        asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(sfw[0]), "=r"(sfw[1]), "=r"(sfw[2]), "=r"(sfw[3])
                     : "l"(sf_row + (uint64_t) it * 16u));
    };
    if (sf_t < n_mma) read_sf(0);
    for (uint32_t it = 0; it < steps; it++) {
      const uint32_t stage = it % kStages, use = it / kStages;
      if (use > 0 && !bar_wait(&sh.empty[stage], (use - 1) & 1u)) {
        sh.fail = 1;
        break;
      }
      const uint32_t st = smem_addr(smem + stage * kStageBytes);
      const uint32_t sa = st, sfa = st + kABytes + kBBytes, sfb = sfa + kSfaBytes;
      // the tokens' scale bytes of the stage (read a stage ahead), a word into each chunk
      if (sf_t < n_mma) {
#pragma unroll
        for (uint32_t ch = 0; ch < kSfChunks; ch++)
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(sfb + (ch * 2u + (sf_t >> 7)) * kChunk + sf_at), "r"(sfw[ch]) : "memory");
        if (it + 1 < steps) read_sf(it + 1);
      }
      // the stage's raw rows have landed (the loader's tensor-map copy): a task = (row, 64 values of K = one MMA's 32
      // bytes of the row), its raw bytes nine aligned words of the row's 144-byte window
      const uint32_t rs = it % kRawStages;
      if (!bar_wait(&sh.raw_full[rs], (it / kRawStages) & 1u)) {
        sh.fail = 1;
        break;
      }
      const uint32_t lead = MX ? 8u * (it & 1u) : 0u;  // (MXFP4: the window starts 8 bytes before an odd stage's bytes)
#pragma unroll
      for (int u = 0; u < kTasks; u++) {
        const uint32_t task = pt + (uint32_t) u * kProdThreads, row = task >> 2, mm = task & 3u;
        const uint32_t off = row * kRawRow + lead + mm * (MX ? 34u : 36u), sh_bits = (off & 3u) * 8u;
        uint32_t r[9];
#pragma unroll
        for (int i = 0; i < 9; i++)
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r[i]) : "r"(raw0 + rs * kRawBytes + (off & ~3u) + 4u * i));
        uint32_t q[8];  // the 64 values' nibbles in K order: 32 bytes
        if constexpr (!MX) {
          // the four scale bytes: ggml reads a byte without its sign bit and 0x7F as zero
          uint32_t s = r[0] & 0x7F7F7F7Fu;
          const uint32_t z = s ^ 0x7F7F7F7Fu;                                // a zero byte where the scale was 0x7F
          const uint32_t hit = ((z - 0x01010101u) & ~z & 0x80808080u) >> 7;  // 1 in such a byte (z's bytes are below 0x80:
          s &= ~(hit * 0xFFu);                                               // a borrow only leaves a byte that is zero)
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(sfa + mm * kChunk + chunk_at(row)), "r"(s) : "memory");
#pragma unroll
          for (int sub = 0; sub < 4; sub++) {
            const uint2 k = k_order16(r[1 + 2 * sub], r[2 + 2 * sub]);
            q[2 * sub] = k.x, q[2 * sub + 1] = k.y;
          }
        } else {
          uint32_t v[9];
#pragma unroll
          for (int i = 0; i < 8; i++) v[i] = __funnelshift_r(r[i], r[i + 1], sh_bits);
          v[8] = r[8] >> sh_bits;
          const uint32_t e0 = v[0] & 0xFFu, e1 = (v[4] >> 8) & 0xFFu;
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(sfa + (mm >> 1) * kChunk + chunk_at(row) + 2u * (mm & 1u)),
                       "h"((uint16_t) (e0 | e1 << 8))
                       : "memory");
#pragma unroll
          for (int b = 0; b < 2; b++) {
            uint32_t c[4];  // the block's 16 bytes: low nibbles values 0 .. 15, high nibbles values 16 .. 31
#pragma unroll
            for (int i = 0; i < 4; i++) c[i] = b ? __funnelshift_r(v[4 + i], v[5 + i], 16) : __funnelshift_r(v[i], v[i + 1], 8);
            const uint2 k0 = k_order16(c[0], c[1]), k1 = k_order16(c[2], c[3]);
            q[4 * b] = k0.x, q[4 * b + 1] = k1.x, q[4 * b + 2] = k0.y, q[4 * b + 3] = k1.y;
          }
        }
        // (a warp's stores: 8 rows x an MMA's two pieces of each - the swizzle spreads them over all the banks)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sa + tile_at(row, 2u * mm)), "r"(q[0]), "r"(q[1]), "r"(q[2]), "r"(q[3]) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sa + tile_at(row, 2u * mm + 1u)), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]) : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these writes before the tensor core's reads
      __syncwarp();
      if (lane == 0) {
        bar_arrive(&sh.full[stage]);
        bar_arrive(&sh.raw_empty[rs]);  // (the warp has read its part of the raw rows)
      }
    }
  } else if (warp == (uint32_t) kRawWarp) {
    // ================= the rows' raw bytes =================
    if (lane == 0) {
      // the rows' raw bytes, a stage's 144-byte window of each of the block's 128 rows a copy, as far ahead as the raw
      // ring is deep (the window of an odd MXFP4 stage starts 8 bytes early, on the 16 bytes a copy must start on)
      const uint32_t raw0 = smem_addr(smem + kStages * kStageBytes);
      for (uint32_t it = 0; it < steps; it++) {
        const uint32_t rs = it % kRawStages, use = it / kRawStages;
        if (use > 0 && !bar_wait(&sh.raw_empty[rs], (use - 1) & 1u)) {
          sh.fail = 1;
          break;
        }
        const uint32_t bar = smem_addr(&sh.raw_full[rs]);
        const uint32_t x = MX ? (it * 136u) & ~15u : it * 144u;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t) kRawBytes) : "memory");
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                         raw0 + rs * kRawBytes),
                     "l"(&wmap), "r"(x), "r"(row0), "r"(bar)
                     : "memory");
      }
    }
  } else if (warp == (uint32_t) kLoaderWarp) {
    // ================= the tokens' codes =================
    if (lane == 0) {
      for (uint32_t it = 0; it < steps; it++) {
        const uint32_t stage = it % kStages, use = it / kStages;
        if (use > 0 && !bar_wait(&sh.empty[stage], (use - 1) & 1u)) {
          sh.fail = 1;
          break;
        }
        const uint32_t bar = smem_addr(&sh.full[stage]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t) kBBytes) : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                smem_addr(smem + stage * kStageBytes + kABytes)),
            "l"(&tmap), "r"(it * 128u), "r"(c0), "r"(bar)
            : "memory");
      }
    }
  } else if (warp == (uint32_t) kIssuerWarp) {
    // ================= issuer =================
    // instruction descriptor (block scaled): A and B E2M1 (format 1), both K-major, N, the scale format, M = 128
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((n_mma >> 3) << 17) | ((MX ? 1u : 0u) << 23) | ((uint32_t) (kM >> 4) << 24);
    // (one lane runs the whole loop: nothing here is the warp's, and the other lanes' polling and the meeting after
    // every stage only stood in its way)
    for (uint32_t it = 0; lane == 0 && it < steps && !sh.fail; it++) {
      const uint32_t stage = it % kStages, use = it / kStages;
      if (!bar_wait(&sh.full[stage], use & 1u)) {
        sh.fail = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      {
        const uint32_t st = smem_addr(smem + stage * kStageBytes);
        // descriptors: everything but the address is the same all along (every address here is below 2^18, so the
        // 14-bit field of address / 16 takes an offset by plain addition)
        constexpr uint64_t kSfDesc = (uint64_t) (16u >> 4) << 16 | (uint64_t) (128u >> 4) << 32 | (uint64_t) 1 << 46;
        constexpr uint64_t kTileDesc = (uint64_t) 1 << 16 | (uint64_t) (1024u >> 4) << 32 | (uint64_t) 1 << 46 | (uint64_t) 2 << 61;
        const uint64_t da0 = kTileDesc | (st >> 4), db0 = kTileDesc | ((st + kABytes) >> 4);
        const uint64_t sfa0 = kSfDesc | ((st + kABytes + kBBytes) >> 4), sfb0 = kSfDesc | ((st + kABytes + kBBytes + kSfaBytes) >> 4);
        // a chunk of scale factors (32 lanes x 16 bytes = 4 columns of tensor memory) for the rows and two for the tokens,
        // then the MMAs that read them: the first MMA of a stage starts after three copies, not twelve
        auto copy_chunk = [&](uint32_t ch) {
          asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfaCol + 4u * ch), "l"(sfa0 + ch * (kChunk >> 4)) : "memory");
          asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfbCol + 8u * ch), "l"(sfb0 + 2u * ch * (kChunk >> 4)) : "memory");
          if (n_mma > 128u)
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfbCol + 8u * ch + 4u),
                         "l"(sfb0 + (2u * ch + 1u) * (kChunk >> 4))
                         : "memory");
        };
#pragma unroll
        for (uint32_t mm = 0; mm < (uint32_t) kMmas; mm++) {
          // both tiles as a tensor-map copy lays the tokens': a row (a token) 128 bytes of K under the 128-byte swizzle, the
          // MMA's 32 bytes of K at 32 mm
          const uint64_t da = da0 + 2u * mm, db = db0 + 2u * mm;
          const uint32_t accumulate = (it | mm) ? 1u : 0u;
          if constexpr (!MX) {  // a chunk a MMA: its four factors are the MMA's four 16s
            copy_chunk(mm);
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmem),
                "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tmem + kSfaCol + 4u * mm), "r"(tmem + kSfbCol + 8u * mm)
                : "memory");
          } else {  // a chunk two MMAs: factors 0, 1 then 2, 3 (the factor id in the descriptor is the first's byte)
            if ((mm & 1u) == 0) copy_chunk(mm >> 1);
            const uint32_t id = 2u * (mm & 1u), idesc_mm = idesc | (id << 4) | (id << 29);
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                " tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmem),
                "l"(da), "l"(db), "r"(idesc_mm), "r"(accumulate), "r"(tmem + kSfaCol + 4u * (mm >> 1)),
                "r"(tmem + kSfbCol + 8u * (mm >> 1))
                : "memory");
          }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&sh.empty[stage])) : "memory");
        if (it + 1 == steps)
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&sh.acc_full)) : "memory");
      }
    }
    __syncwarp();
  } else {
    // ================= epilogue =================
    const uint32_t row = 32u * warp + lane;  // this thread's weight row of the tile = its TMEM lane
    const uint32_t lane_base = tmem + ((32u * warp) << 16);
    float* y = a.y + (uint64_t) c0 * a.ys + row0 + row;
    if (bar_wait(&sh.acc_full, 0)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (uint32_t col = 0; col < n_mma; col += 32) {
        uint32_t r[32];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
              "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(lane_base + col)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; i++)
          if (col + i < n_valid) y[(uint64_t) (col + i) * a.ys] = mul_rn(__uint_as_float(r[i]), a.scale);
      }
    } else {
      sh.fail = 1;
    }
  }
  // ================= common exit =================
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == (uint32_t) kIssuerWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
  if (tid == 0 && sh.fail) atomicOr(a.status, 1u);
}

uint32_t* status_word() {
  static uint32_t* at[64];
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
  if (!at[d]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
    at[d] = (uint32_t*) p;
  }
  return at[d];
}

// the driver's tensor-map encoder, looked up once (no link against the driver library)
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled) p;
  }
  return fn;
}

// the tokens' codes as [token][byte] (n rows of cols / 2 bytes, a row `stride` bytes on): a box of 256 tokens x 128 bytes (a
// stage's K), written with the 128-byte swizzle the MMA's B descriptor names; tokens past the last are filled with zeros
bool codes_map(const void* aq, uint32_t n, uint32_t cols, uint32_t stride, CUtensorMap* tm) {
  const EncodeTiled enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {cols / 2, n};
  const cuuint64_t strides[1] = {stride};
  const cuuint32_t box[2] = {128, (cuuint32_t) kNMax}, unit[2] = {1, 1};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(aq), dims, strides, box, unit, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// the weight matrix as [row][byte]: a box of 128 rows x 144 bytes (a stage's raw bytes of each row)
bool rows_map(const void* w, uint32_t rows, uint64_t row_bytes, CUtensorMap* tm) {
  const EncodeTiled enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t) kRawRow, (cuuint32_t) kM}, unit[2] = {1, 1};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), dims, strides, box, unit, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool MX>
int launch(const Args& a, cudaStream_t s) {
  alignas(64) CUtensorMap tmap, wmap;
  memset(&tmap, 0, sizeof tmap), memset(&wmap, 0, sizeof wmap);
  const uint64_t row_bytes = MX ? (uint64_t) (a.cols / 32) * 17 : (uint64_t) (a.cols / 64) * 36;
  if (!codes_map(a.aq, a.n, a.cols, a.aq_stride, &tmap) || !rows_map(a.w, a.rows, row_bytes, &wmap)) return 0;
  static bool sized[64] = {};  // (one record a template instance, one flag a device)
  const int smem_bytes = kStages * kStageBytes + kRawStages * kRawBytes;
  if (!allow_dynamic_smem(fp4_tc_kernel<MX>, smem_bytes, sized)) return 0;
  const dim3 grid(a.rows / kM, (a.n + kNMax - 1) / kNMax);
  fp4_tc_kernel<MX><<<grid, kThreads, smem_bytes, s>>>(a, tmap, wmap);
  return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace

uint32_t instr_desc(bool mx, uint32_t n, uint32_t sf_id) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((mx ? 1u : 0u) << 23) | ((uint32_t) (kM >> 4) << 24) | (sf_id << 4) | (sf_id << 29);
}

int try_launch(bool mx, const void* w, uint32_t rows, uint32_t cols, const void* aq, uint32_t aq_stride, const void* as,
               uint32_t as_stride, uint32_t n, float scale, float* y, uint32_t ys, void* stream) {
  // whole 128-row tiles and 256-value steps; the tokens' codes copied 16 bytes at a time, a stage's scale bytes of a token read by one load
  if (!rows || rows % kM || !cols || cols % kStepValues || !n) return 0;
  if (((uintptr_t) aq & 15u) || aq_stride % 16u || ((uintptr_t) as & (mx ? 7u : 15u)) || as_stride % (mx ? 8u : 16u)) return 0;
  // the rows' raw bytes come by tensor-map copies: the matrix and its rows start on 16 bytes (a row of whole 256-value
  // steps is 144 or 136 bytes a step: cols in 512s gives MXFP4 rows of whole 16s)
  if (((uintptr_t) w & 15u) || (mx ? (uint64_t) (cols / 32) * 17 : (uint64_t) (cols / 64) * 36) % 16u) return 0;
  uint32_t* status = status_word();
  if (!status) return 0;
  const Args a{(const uint8_t*) w, (const uint8_t*) aq, (const uint8_t*) as, y, rows, cols, n, ys, aq_stride, as_stride, scale, status};
  return mx ? launch<true>(a, (cudaStream_t) stream) : launch<false>(a, (cudaStream_t) stream);
}

uint32_t read_status() {
  uint32_t* at = status_word();
  if (!at) return 0x80000000u;
  uint32_t v = 0, zero = 0;
  if (cudaMemcpy(&v, at, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return 0x80000000u;
  cudaMemcpy(at, &zero, sizeof zero, cudaMemcpyHostToDevice);
  return v;
}

}  // namespace fp4_tc
}  // namespace osmos
