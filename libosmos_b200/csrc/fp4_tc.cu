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
//                        the scale-factor chunk layout (128 rows x 4 factors: byte (r % 32) * 16 + (r / 32) * 4 + f);
//                        the tokens' codes and scales are already in K order and go to the same layouts by cp.async.
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

#include "common.cuh"

namespace osmos {
namespace fp4_tc {
namespace {

constexpr int kM = 128, kNMax = 256;
constexpr int kEpiWarps = 4, kProdWarps = 8;
constexpr int kIssuerWarp = kEpiWarps;
constexpr int kFirstProdWarp = kEpiWarps + 1;
constexpr int kProdThreads = kProdWarps * kWarp;
constexpr int kThreads = (kEpiWarps + 1 + kProdWarps) * kWarp;
constexpr int kStages = 4;
constexpr int kStepValues = 256, kMmaK = 64, kMmas = kStepValues / kMmaK;  // a stage: 256 values of K, four MMAs
constexpr int kABytes = kM * kStepValues / 2;                              // 16 KB: 4 MMA tiles of 128 rows x 32 bytes
constexpr int kBBytes = kNMax * kStepValues / 2;                           // 32 KB
constexpr int kChunk = 512;                                                // a scale-factor chunk: 128 rows x 4 factors
constexpr int kSfaBytes = 4 * kChunk, kSfbBytes = 2 * 4 * kChunk;          // at most 4 chunks of K a stage; B: two row halves
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;     // 54 KB
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
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// shared-memory matrix descriptor: K-major, no swizzle, core matrices of 8 rows x 16 bytes; lbo: to the next 16 bytes of
// K, sbo: to the next 8 rows (cute/arch/mma_sm100_desc.hpp: start >> 4, leading >> 4 at bit 16, stride >> 4 at bit 32,
// version 1 at bit 46, layout type 0)
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) (lbo_bytes >> 4) << 16 | (uint64_t) (sbo_bytes >> 4) << 32 |
         (uint64_t) 1 << 46;
}

// where row r's 16 bytes `half` (0, 1) of an MMA's 32 bytes of K lie in an operand tile
__device__ __forceinline__ uint32_t tile_at(uint32_t r, uint32_t half) { return (r >> 3) * 256u + half * 128u + (r & 7u) * 16u; }
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
  uint64_t full[kStages], empty[kStages], acc_full;
  uint32_t tmem_base;
  int fail;
};

// MX false: NVFP4 (a 36-byte block of 64 values: 4 UE4M3 bytes, then 8 bytes a 16); MX true: MXFP4 (a 17-byte block of
// 32 values: the E8M0 byte, then 16 bytes)
template <bool MX>
__global__ void __launch_bounds__(kThreads, 1) fp4_tc_kernel(const Args a) {
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
    for (int i = 0; i < kStages; i++) bar_init(&sh.full[i], kProdThreads), bar_init(&sh.empty[i], 1);
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

  if (warp >= (uint32_t) kFirstProdWarp) {
    // ================= producers =================
    const uint32_t pt = tid - kFirstProdWarp * kWarp;
    for (uint32_t it = 0; it < steps; it++) {
      const uint32_t stage = it % kStages, use = it / kStages;
      if (use > 0 && !bar_wait(&sh.empty[stage], (use - 1) & 1u)) {
        sh.fail = 1;
        break;
      }
      const uint32_t st = smem_addr(smem + stage * kStageBytes);
      const uint32_t sa = st, sb = st + kABytes, sfa = sb + kBBytes, sfb = sfa + kSfaBytes;
      // B: a token's 128 bytes of codes as 8 pieces of 16 (MMA m's halves 0, 1), its scale bytes a chunk's word at a time
      for (uint32_t i = pt; i < n_mma * 8u; i += kProdThreads) {
        const uint32_t t = i >> 3, piece = i & 7u, tok = c0 + (t < n_valid ? t : n_valid - 1);
        cp_async16(sb + (piece >> 1) * (kNMax * 32u) + tile_at(t, piece & 1u),
                   a.aq + (uint64_t) tok * a.aq_stride + (uint64_t) it * 128u + piece * 16u);
      }
      for (uint32_t i = pt; i < n_mma * kSfChunks; i += kProdThreads) {
        const uint32_t t = i / kSfChunks, ch = i % kSfChunks, tok = c0 + (t < n_valid ? t : n_valid - 1);
        cp_async4(sfb + (ch * 2u + (t >> 7)) * kChunk + chunk_at(t & 127u),
                  a.as + (uint64_t) tok * a.as_stride + (uint64_t) it * (kSfChunks * 4u) + ch * 4u);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      // A: a task = (row, 64 values of K = one MMA's 32 bytes of the row)
      for (uint32_t task = pt; task < (uint32_t) (kM * kMmas); task += kProdThreads) {
        const uint32_t row = task >> 2, mm = task & 3u;
        uint32_t q[8];  // the 64 values' nibbles in K order: 32 bytes
        if constexpr (!MX) {
          const uint32_t* blk = (const uint32_t*) (a.w + (uint64_t) (row0 + row) * row_bytes + ((uint64_t) it * 4u + mm) * 36u);
          uint32_t r[9];
#pragma unroll
          for (int i = 0; i < 9; i++) r[i] = __ldg(blk + i);
          // the four scale bytes: ggml reads a byte without its sign bit and 0x7F as zero
          uint32_t s = r[0] & 0x7F7F7F7Fu;
          const uint32_t z = s ^ 0x7F7F7F7Fu;                                  // a zero byte where the scale was 0x7F
          const uint32_t hit = ((z - 0x01010101u) & ~z & 0x80808080u) >> 7;    // 1 in such a byte (no borrow can reach a
          s &= ~(hit * 0xFFu);                                                 // byte above a non-zero one falsely: z < 0x80)
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(sfa + mm * kChunk + chunk_at(row)), "r"(s) : "memory");
#pragma unroll
          for (int sub = 0; sub < 4; sub++) {
            const uint2 k = k_order16(r[1 + 2 * sub], r[2 + 2 * sub]);
            q[2 * sub] = k.x, q[2 * sub + 1] = k.y;
          }
        } else {
          // two 17-byte blocks (34 bytes) that start 2 mod 4 bytes into a word for every other pair
          const uint64_t off = (uint64_t) (row0 + row) * row_bytes + ((uint64_t) it * 4u + mm) * 34u;
          const uint32_t* al = (const uint32_t*) (a.w + (off & ~(uint64_t) 3));
          const uint32_t shb = (uint32_t) (off & 3u) * 8u;
          uint32_t r[10];
#pragma unroll
          for (int i = 0; i < 9; i++) r[i] = __ldg(al + i);
          r[9] = 0;
          uint32_t v[9];
#pragma unroll
          for (int i = 0; i < 9; i++) v[i] = __funnelshift_r(r[i], r[i + 1], shb);
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
        const uint32_t at = sa + mm * (kM * 32u);
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(at + tile_at(row, 0)), "r"(q[0]), "r"(q[1]), "r"(q[2]), "r"(q[3]) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(at + tile_at(row, 1)), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]) : "memory");
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these writes before the tensor core's reads
      bar_arrive(&sh.full[stage]);
    }
  } else if (warp == (uint32_t) kIssuerWarp) {
    // ================= issuer =================
    // instruction descriptor (block scaled): A and B E2M1 (format 1), both K-major, N, the scale format, M = 128
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((n_mma >> 3) << 17) | ((MX ? 1u : 0u) << 23) | ((uint32_t) (kM >> 4) << 24);
    for (uint32_t it = 0; it < steps && !sh.fail; it++) {
      const uint32_t stage = it % kStages, use = it / kStages;
      if (!bar_wait(&sh.full[stage], use & 1u)) {
        sh.fail = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint32_t st = smem_addr(smem + stage * kStageBytes);
        const uint32_t sa = st, sb = st + kABytes, sfa = sb + kBBytes, sfb = sfa + kSfaBytes;
        // the stage's scale factors into tensor memory: a chunk = 32 lanes x 16 bytes = 4 columns
        for (uint32_t ch = 0; ch < kSfChunks; ch++) {
          asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfaCol + 4u * ch),
                       "l"(tile_desc(sfa + ch * kChunk, 16, 128))
                       : "memory");
          asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfbCol + 8u * ch),
                       "l"(tile_desc(sfb + (ch * 2u) * kChunk, 16, 128))
                       : "memory");
          if (n_mma > 128u)
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfbCol + 8u * ch + 4u),
                         "l"(tile_desc(sfb + (ch * 2u + 1u) * kChunk, 16, 128))
                         : "memory");
        }
        for (uint32_t mm = 0; mm < (uint32_t) kMmas; mm++) {
          const uint64_t da = tile_desc(sa + mm * (kM * 32u), 128, 256), db = tile_desc(sb + mm * (kNMax * 32u), 128, 256);
          const uint32_t accumulate = (it | mm) ? 1u : 0u;
          if constexpr (!MX) {  // a chunk a MMA: its four factors are the MMA's four 16s
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmem),
                "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tmem + kSfaCol + 4u * mm), "r"(tmem + kSfbCol + 8u * mm)
                : "memory");
          } else {  // a chunk two MMAs: factors 0, 1 then 2, 3 (the factor id in the descriptor is the first's byte)
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
      __syncwarp();
    }
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

template <bool MX>
int launch(const Args& a, cudaStream_t s) {
  static bool sized[64] = {};  // (one record a template instance, one flag a device)
  const int smem_bytes = kStages * kStageBytes;
  if (!allow_dynamic_smem(fp4_tc_kernel<MX>, smem_bytes, sized)) return 0;
  const dim3 grid(a.rows / kM, (a.n + kNMax - 1) / kNMax);
  fp4_tc_kernel<MX><<<grid, kThreads, smem_bytes, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace

uint32_t instr_desc(bool mx, uint32_t n, uint32_t sf_id) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((mx ? 1u : 0u) << 23) | ((uint32_t) (kM >> 4) << 24) | (sf_id << 4) | (sf_id << 29);
}

int try_launch(bool mx, const void* w, uint32_t rows, uint32_t cols, const void* aq, uint32_t aq_stride, const void* as,
               uint32_t as_stride, uint32_t n, float scale, float* y, uint32_t ys, void* stream) {
  // whole 128-row tiles and 256-value steps; the tokens' rows copied 16 bytes (codes) and 4 bytes (scales) at a time
  if (!rows || rows % kM || !cols || cols % kStepValues || !n) return 0;
  if (((uintptr_t) aq & 15u) || aq_stride % 16u || ((uintptr_t) as & 3u) || as_stride % 4u) return 0;
  if (mx ? ((uintptr_t) w & 3u) != 0 || (cols / 32 * 17) % 4u != 0 : ((uintptr_t) w & 3u) != 0) return 0;
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
