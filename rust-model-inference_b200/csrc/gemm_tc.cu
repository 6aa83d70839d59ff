// Q8_0 x Q8_0 prefill GEMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// out[m, n] = sum over 32-blocks b of  f16(w.d[n,b]) * xs[m,b] * (int32 dot of block b)
// accumulated in block order exactly as the reference's whole-block variants do:
//   NEON    sum = fma(f32(dot), wd*xs, sum)     src/ops/kernel/q8_0/neon.rs:59-70
//   SCALAR  sum += (wd*xs) * f32(dot)           src/ops/kernel/q8_0/scalar.rs:42-56
//
// tcgen05.mma.kind::i8 has K = 32 per instruction = one Q8_0 block, so every MMA writes a
// fresh 128 x NT int32 tile into tensor memory (two buffers of four blocks each) and the
// epilogue warps drain it (tcgen05.ld), rescale and accumulate in f32 registers while the
// MMAs of the next K slab run.
//
// Roles (576 threads): warp 0 = bulk-copy producer (cp.async.bulk into a 4-stage ring of
// 128-byte K slabs: A image, B image, both scale slabs), warp 1 = TMEM owner + single-thread
// MMA issuer, warps 2..17 = epilogue (warp w may touch TMEM lanes 32*(w%4).., the four warps
// of a lane quadrant split the tile columns).  The epilogue math is packed two columns per
// instruction (mul/fma.rn.f32x2), each half rounded exactly like the scalar instruction.
//
// Operands arrive pre-tiled in HBM in the tcgen05 K-major no-swizzle core-matrix order
// (8 rows x 16 B, LBO = 128 B along K, SBO = 1024 B along rows), so a stage is filled by
// contiguous bulk copies and no tensor map is needed.
//
// The kernel is persistent: one CTA per SM walks the output tiles, the barrier phases run on
// across tiles, so the bulk copies and MMAs of the next tile overlap the tail of the current one.
//
// Every wait is bounded: after the context's wait limit (two seconds by default) of failed polls a role records a site id in the
// context's status word, raises a shared abort flag that all other waits observe, and the
// CTA falls through to the common teardown (TMEM is always deallocated).
#include "common.cuh"
#include "kernels.cuh"

namespace {

constexpr int STAGES = 4;
constexpr int SLAB_BYTES_A = 128 * 128;  // 128 rows x 128 B of K
constexpr int NBUF = 4;
constexpr uint32_t WAIT_LIMIT = 1u << 26;

struct gemm_params {
  const uint8_t* a_img;
  const float* a_scales;
  const uint8_t* b_img;
  const float* b_scales;
  size_t m, n_rows_w, blocks, n_slabs;
  size_t col_begin, col_end;
  float* out;
  size_t out_stride;
  size_t n_ff;
  uint8_t* act_img;
  float* act_scales;
  float* act_f32;
  int32_t* sums;
  size_t n_tiles_n;
  size_t n_tiles;  // m_tiles * n_tiles_n; CTAs walk tiles blockIdx.x, +gridDim.x, ...
  size_t act_slabs, act_blocks;
  rmi_dev_status* status;
  out_fanout fo;  // extra copies of the f32 output (GEMM_EPI_F32)
  int transpose;  // GEMM_EPI_F32: store element (row, n) at out[n * out_stride + row]
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// K-major, no swizzle: LBO = 128 B (next 16-byte K chunk), SBO = 1024 B (next 8 rows)
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint32_t lo = ((saddr >> 4) & 0x3FFFu) | (((128u >> 4) & 0x3FFFu) << 16);
  uint32_t hi = ((1024u >> 4) & 0x3FFFu) | (1u << 14);  // descriptor version 1 (sm_100)
  return ((uint64_t)hi << 32) | lo;
}

template <int NT>
__device__ __forceinline__ constexpr uint32_t umma_idesc_i8() {
  // D = s32 (2 @ bit 4), A = B = signed 8-bit (1 @ bits 7, 10), K-major both, N/8 @ 17, M/16 @ 24
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u), "r"(0u)
      : "memory");
}

// The four MMAs of one K slab (blocks 0..3: operand start addresses 256 B apart, accumulators NT columns apart).
template <int NT>
__device__ __forceinline__ void umma_i8_x4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b32 z, d1, d2, d3;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "mov.b32 z, 0;\n\t"
      "setp.ne.b32 p, z, 0;\n\t"
      "add.u32 d1, %0, %4;\n\tadd.u32 d2, d1, %4;\n\tadd.u32 d3, d2, %4;\n\t"
      "add.u64 a1, %1, 16;\n\tadd.u64 a2, %1, 32;\n\tadd.u64 a3, %1, 48;\n\t"
      "add.u64 b1, %2, 16;\n\tadd.u64 b2, %2, 32;\n\tadd.u64 b3, %2, 48;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {z, z, z, z}, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [d1], a1, b1, %3, {z, z, z, z}, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [d2], a2, b2, %3, {z, z, z, z}, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [d3], a3, b3, %3, {z, z, z, z}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)NT)
      : "memory");
}

__device__ __forceinline__ void umma_commit_a(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- packed f32x2 arithmetic (two independent IEEE round-to-nearest operations) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float* lo, float* hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, int* r);
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, int* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, int* r) {
  tmem_ld16(taddr, r);
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

constexpr int EPI_WARPS = 16;
constexpr int THREADS = 64 + EPI_WARPS * 32;

struct __align__(128) smem_layout_hdr {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tfull[NBUF];
  uint64_t tempty[NBUF];
  uint32_t tmem_base;
  int abort_flag;
};

// Per-stage shared memory: A image (16 KiB) | B image (NT*128 B) | weight scales [4][128] f32 |
// activation scales [4][128] f32.
template <int NT>
struct stage_layout {
  static constexpr int A = 0;
  static constexpr int B = SLAB_BYTES_A;
  static constexpr int WS = B + NT * 128;
  static constexpr int XS = WS + 4 * 128 * 4;  // the weight tile's scales of all 128 rows: one contiguous copy
  static constexpr int BYTES = XS + 4 * 128 * 4;
};

// Out-of-line slow path of a wait: keeps polling with the time limit, records the failure.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar_addr, uint32_t parity, volatile int* abort_flag,
                                            rmi_dev_status* status, int site, int detail) {
  // The common case is a phase that completes during the first suspended tries: the global timer (a slow
  // read) and the abort flag are only consulted after every eighth failed try.
  uint64_t t0 = 0;
  const uint64_t limit_ns = status->limit_ns;
  for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar_addr), "r"(parity), "r"(20000u)
        : "memory");
    if (ok) return true;
    if ((i & 7) == 7) {
      if (*abort_flag) return false;
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) break;
    }
  }
  *abort_flag = 1;
  if (atomicCAS(&status->code, 0, RMI_ERR_TIMEOUT) == 0) {
    status->where = site;
    status->detail = detail;
  }
  return false;
}

// Hot path of a bounded wait: one try (the hardware suspends the thread until the phase
// completes or a time slice passes), then the slow path.
__device__ __forceinline__ bool mbar_wait_a(uint32_t bar_addr, uint32_t parity, volatile int* abort_flag,
                                            rmi_dev_status* status, int site, int detail) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar_addr), "r"(parity), "r"(20000u)
      : "memory");
  if (ok) return true;
  return mbar_wait_slow(bar_addr, parity, abort_flag, status, site, detail);
}

__device__ __forceinline__ void mbar_arrive_a(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}

// NT: tile columns (32 or 64).  EPI: GEMM_EPI_*.  SEM: RMI_SEM_NEON, RMI_SEM_SCALAR, or RMI_SEM_AVX2 (x86
// quantizer in the SwiGLU epilogue, whole-block fma accumulate).
// Tensor memory holds two slab buffers of four K-blocks each (2 * 4 * NT columns): the MMA
// warp fills one slab buffer (four MMAs, one commit) while the epilogue drains the other,
// so barriers are exchanged once per 128-byte K slab instead of once per block.
// For GEMM_EPI_SWIGLU_Q8 (NT = 64) the weight is in the gate/up-interleaved order: rows
// [64t, 64t+32) are gate columns 32t.., rows [64t+32, 64t+64) the matching up columns.
template <int NT, int EPI, int SEM>
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_kernel(const gemm_params p) {
  using SL = stage_layout<NT>;
  constexpr int CPW = NT / 4;  // columns per epilogue warp
  // tensor-memory slab buffers (four K blocks each): as many as fit in 512 columns, so that more MMA groups
  // are in flight while a finished one waits for the epilogue
#ifndef RMI_TMEM_BUFS32
#define RMI_TMEM_BUFS32 4
#endif
  constexpr int NB = NT == 32 ? RMI_TMEM_BUFS32 : 2;
  constexpr uint32_t TMEM_COLS = NB * 4 * NT;
  static_assert(TMEM_COLS <= 512 && CPW >= 8, "tile width must be 32 or 64");
  extern __shared__ __align__(128) uint8_t smem_raw[];
  smem_layout_hdr* hdr = reinterpret_cast<smem_layout_hdr*>(smem_raw);
  uint8_t* stages = smem_raw + 1024;
  volatile int* abort_flag = &hdr->abort_flag;
  const uint32_t full_a = smem_u32(&hdr->full[0]), empty_a = smem_u32(&hdr->empty[0]);
  const uint32_t tfull_a = smem_u32(&hdr->tfull[0]), tempty_a = smem_u32(&hdr->tempty[0]);
  const uint32_t stages_a = smem_u32(stages);

  const int warp = threadIdx.x / 32, lane = threadIdx.x & 31;
  const int n_tiles = (int)p.n_tiles, n_tiles_n = (int)p.n_tiles_n;
  const int n_slabs = (int)p.n_slabs, blocks = (int)p.blocks;
  constexpr bool kScales = EPI != GEMM_EPI_BLOCK_SUMS;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; i++) {
      mbar_init(&hdr->full[i], 1);
      mbar_init(&hdr->empty[i], 1 + EPI_WARPS);
    }
    for (int i = 0; i < NB; i++) {
      mbar_init(&hdr->tfull[i], 1);
      mbar_init(&hdr->tempty[i], EPI_WARPS);
    }
    hdr->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hdr->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  // Dependent launch: barriers and tensor memory are set up while the preceding kernel drains; everything below
  // reads what it wrote (activation images and scales) or writes what it may still read.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // Lanes 0..3 each own one of the stage's four bulk copies (A image, B image, weight scales, activation
    // scales), so a slab costs one short instruction stream for the whole warp: the roles that run on a single
    // warp set the pace of the pipeline and compete with sixteen epilogue warps for issue slots.
    if (lane < (kScales ? 4 : 2)) {
      int gs = 0;  // slabs issued so far (all tiles)
      const uint32_t dst_off = lane == 0 ? SL::A : (lane == 1 ? SL::B : (lane == 2 ? SL::WS : SL::XS));
      const uint32_t full_bytes = lane == 0 ? SLAB_BYTES_A : (lane == 1 ? NT * 128 : 4 * 512);
      const size_t stride = lane < 2 ? (size_t)SLAB_BYTES_A : (size_t)4 * 512;  // bytes from one slab's source to the next
      const int last_kb = blocks - (n_slabs - 1) * 4;                           // blocks in the last slab (1..4)
      const uint32_t last_bytes = lane < 2 ? full_bytes : (uint32_t)last_kb * 512;
      const uint32_t tx_full = SLAB_BYTES_A + NT * 128 + (kScales ? 4 * 1024 : 0);
      const uint32_t tx_last = SLAB_BYTES_A + NT * 128 + (kScales ? (uint32_t)last_kb * 1024 : 0);
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int tile_n = tile % n_tiles_n, tile_m = tile / n_tiles_n;
        const size_t wrow_tile = p.col_begin + (size_t)tile_n * NT;
        const uint8_t* src;
        if (lane == 0) src = p.a_img + (size_t)tile_m * p.n_slabs * SLAB_BYTES_A;
        else if (lane == 1) src = p.b_img + (wrow_tile / 128) * p.n_slabs * SLAB_BYTES_A + ((wrow_tile % 128) / 8) * 1024;
        else if (lane == 2) src = reinterpret_cast<const uint8_t*>(p.b_scales + (wrow_tile / 128) * p.blocks * 128);
        else src = reinterpret_cast<const uint8_t*>(p.a_scales + (size_t)tile_m * p.blocks * 128);
        for (int s = 0; s < n_slabs; s++, gs++, src += stride) {
          const int st = gs % STAGES;
          if (gs >= STAGES && !mbar_wait_a(empty_a + 8 * st, ((gs / STAGES) & 1) ^ 1, abort_flag, p.status, 1, s)) {
            tile = n_tiles;
            break;
          }
          const bool last = s + 1 == n_slabs;
          const uint32_t bar = full_a + 8 * st;
          if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(last ? tx_last : tx_full)
                         : "memory");
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           stages_a + (uint32_t)(st * SL::BYTES) + dst_off),
                       "l"(src), "r"(last ? last_bytes : full_bytes), "r"(bar)
                       : "memory");
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8<NT>();
      // descriptors differ from stage to stage and block to block only in the 14-bit start address field
      const uint64_t adesc0 = umma_desc(stages_a + SL::A), bdesc0 = umma_desc(stages_a + SL::B);
      int gs = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x)
      for (int s = 0; s < n_slabs; s++, gs++) {
        const int st = gs % STAGES, tb = gs % NB;
        if (!mbar_wait_a(full_a + 8 * st, (gs / STAGES) & 1, abort_flag, p.status, 2, s) ||
            (gs >= NB && !mbar_wait_a(tempty_a + 8 * tb, ((gs / NB) & 1) ^ 1, abort_flag, p.status, 3, s))) {
          tile = n_tiles;
          break;
        }
        tc_fence_after();
        const uint64_t so = (uint64_t)((st * SL::BYTES) >> 4);
        const uint32_t d0 = tmem_base + (uint32_t)(tb * 4 * NT);
        if (s + 1 < n_slabs || (blocks & 3) == 0) {
          umma_i8_x4<NT>(d0, adesc0 + so, bdesc0 + so, idesc);
        } else {
          const int kb_n = blocks - s * 4;
          for (int kb = 0; kb < kb_n; kb++)
            umma_i8(d0 + (uint32_t)(kb * NT), adesc0 + so + (uint64_t)(kb * 16), bdesc0 + so + (uint64_t)(kb * 16), idesc);
        }
        umma_commit_a(tfull_a + 8 * tb);  // the slab's accumulators are complete
        umma_commit_a(empty_a + 8 * st);  // A/B of this stage have been read
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (16 warps)
    const int q = warp % 4;             // TMEM lane quadrant this warp may access
    const int cg = (warp - 2) / 4;      // which quarter of the tile columns
    const int r_tile = q * 32 + lane;   // row inside the 128-row tile
    const int col0 = cg * CPW;
    const uint32_t tmem_lane = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col0;
    bool ok = true;
    int gs = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
    const int tile_n = tile % n_tiles_n, tile_m = tile / n_tiles_n;
    const size_t wrow_tile = p.col_begin + (size_t)tile_n * NT;
    const size_t row = (size_t)tile_m * 128 + r_tile;
    const int ws_col = (int)(wrow_tile % 128) + col0;  // this thread's first column inside the 128-row weight tile
    uint64_t acc[CPW / 2];
#pragma unroll
    for (int c = 0; c < CPW / 2; c++) acc[c] = 0ull;

    for (int s = 0; s < n_slabs; s++, gs++) {
      const int st = gs % STAGES, tb = gs % NB;
      const uint8_t* sb = stages + st * SL::BYTES;
      const int kb_n = blocks - s * 4 < 4 ? blocks - s * 4 : 4;
      // tfull[tb] completes after the MMAs of slab s, which were issued after full[st] completed;
      // waiting on full[st] as well makes the bulk-copied scale slabs visible to this thread.
      if (kScales && !mbar_wait_a(full_a + 8 * st, (gs / STAGES) & 1, abort_flag, p.status, 5, s)) {
        ok = false;
        break;
      }
      if (!mbar_wait_a(tfull_a + 8 * tb, (gs / NB) & 1, abort_flag, p.status, 4, s)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int half = 0; half < 2; half++) {
        int d[2][CPW];
        tmem_ld<CPW>(tmem_lane + (uint32_t)((tb * 4 + half * 2) * NT), d[0]);
        tmem_ld<CPW>(tmem_lane + (uint32_t)((tb * 4 + half * 2 + 1) * NT), d[1]);
        tmem_ld_wait();
        if (half == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_a(tempty_a + 8 * tb);  // slab buffer back to the MMA warp
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int kb = half * 2 + j;
          if (kb < kb_n) {
            if (EPI == GEMM_EPI_BLOCK_SUMS) {
              if (row < p.m) {
#pragma unroll
                for (int c = 0; c < CPW; c++) {
                  const size_t n = wrow_tile + col0 + c;
                  if (n < p.col_end) p.sums[(row * p.n_rows_w + n) * p.blocks + (size_t)(s * 4 + kb)] = d[j][c];
                }
              }
            } else {
              const float xs = reinterpret_cast<const float*>(sb + SL::XS)[kb * 128 + r_tile];
              const uint64_t* wsp = reinterpret_cast<const uint64_t*>(sb + SL::WS + (kb * 128 + ws_col) * 4);
              const uint64_t xs2 = pack2(xs, xs);
#pragma unroll
              for (int c = 0; c < CPW / 2; c++) {
                const uint64_t s2 = mul2(wsp[c], xs2);
                const uint64_t f2 = pack2(__int2float_rn(d[j][2 * c]), __int2float_rn(d[j][2 * c + 1]));
                if (SEM == RMI_SEM_SCALAR) {
                  // scalar.rs:55: separate multiply and add.  Written with scalar instructions: the
                  // packed mul/add pair did not reproduce the two roundings on the device.
                  float s_lo, s_hi, f_lo, f_hi, a_lo, a_hi;
                  unpack2(s2, &s_lo, &s_hi);
                  unpack2(f2, &f_lo, &f_hi);
                  unpack2(acc[c], &a_lo, &a_hi);
                  acc[c] = pack2(__fadd_rn(a_lo, __fmul_rn(s_lo, f_lo)), __fadd_rn(a_hi, __fmul_rn(s_hi, f_hi)));
                } else {
                  acc[c] = fma2(f2, s2, acc[c]);  // neon.rs:69
                }
              }
            }
          }
        }
      }
      // this warp no longer reads the stage's scale slabs
      __syncwarp();
      if (lane == 0) mbar_arrive_a(empty_a + 8 * st);
    }

    if (EPI == GEMM_EPI_F32 && ok) {
      if (row < p.m && p.transpose) {
        // operands swapped: `row` is a weight row, the tile's columns are activation rows; consecutive
        // lanes store consecutive addresses
        const size_t n0 = wrow_tile + col0;
        float v[CPW];
#pragma unroll
        for (int c = 0; c < CPW / 2; c++) unpack2(acc[c], &v[2 * c], &v[2 * c + 1]);
#pragma unroll
        for (int c = 0; c < CPW; c++)
          if (n0 + c < p.col_end) store_fanout(p.out + (n0 + c) * p.out_stride + row, v[c], p.fo);
      } else if (row < p.m) {
        const size_t n0 = wrow_tile + col0;
        float* o = p.out + row * p.out_stride + n0;
        float v[CPW];
#pragma unroll
        for (int c = 0; c < CPW / 2; c++) unpack2(acc[c], &v[2 * c], &v[2 * c + 1]);
#pragma unroll
        for (int copy = 0; copy < RMI_MAX_FANOUT; copy++) {
          if (copy > p.fo.n) break;
          if (copy > 0) o = reinterpret_cast<float*>(reinterpret_cast<char*>(p.out + row * p.out_stride + n0) + p.fo.delta[copy - 1]);
          if (n0 + CPW <= p.col_end && ((p.out_stride | n0) & 3) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
            for (int c = 0; c < CPW; c += 4) *reinterpret_cast<float4*>(o + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
          } else {
#pragma unroll
            for (int c = 0; c < CPW; c++)
              if (n0 + c < p.col_end) o[c] = v[c];
          }
        }
      }
    }
    if (EPI == GEMM_EPI_SWIGLU_Q8) {
      // [128][65] f32 exchange buffer behind the stage ring (gate columns 0..31, up columns 32..63)
      float* fin = reinterpret_cast<float*>(stages + STAGES * SL::BYTES);
      epi_bar_sync();  // the previous tile's readers are done with the buffer
      if (*abort_flag) ok = false;  // read after the barrier: every epilogue warp leaves at the same tile
#pragma unroll
      for (int c = 0; c < CPW / 2; c++) {
        float a, b;
        unpack2(acc[c], &a, &b);
        fin[r_tile * 65 + col0 + 2 * c] = a;
        fin[r_tile * 65 + col0 + 2 * c + 1] = b;
      }
      epi_bar_sync();
      // src/ops/activation/mod.rs:137-151 then the Q8_0 quantizer: 4 threads per row, 8 columns each;
      // the tile's 32 activation columns are exactly one Q8_0 block of the FFN activation.
      const int e = threadIdx.x - 64;
      const int fr = e / 4, sub = e % 4;
      float v[8];
      float amax = 0.0f;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        const float gte = fin[fr * 65 + sub * 8 + c], up = fin[fr * 65 + 32 + sub * 8 + c];
        const float sl = __fdiv_rn(gte, __fadd_rn(1.0f, exp_cr(-gte)));
        v[c] = __fmul_rn(up, sl);
        amax = fmaxf(amax, fabsf(v[c]));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      float dsc, inv;
      q8_scale_pair<SEM>(amax, &dsc, &inv);
      const size_t k0 = (wrow_tile / 64) * 32 + sub * 8;  // column inside n_ff
      const size_t frow = (size_t)tile_m * 128 + fr;
      if (ok) {
        if (p.act_f32 && frow < p.m) {
#pragma unroll
          for (int c = 0; c < 8; c++) p.act_f32[frow * p.n_ff + k0 + c] = v[c];
        }
        uint32_t pk[2] = {0u, 0u};
#pragma unroll
        for (int c = 0; c < 8; c++) pk[c / 4] |= (uint32_t)(uint8_t)(int8_t)q8_quant_value<SEM>(v[c], inv) << (8 * (c % 4));
        uint8_t* img = p.act_img + ((size_t)tile_m * p.act_slabs + k0 / 128) * SLAB_BYTES_A + (fr / 8) * 1024 +
                       (fr % 8) * 16 + ((k0 % 128) / 16) * 128 + (k0 % 16);
        *reinterpret_cast<uint2*>(img) = make_uint2(pk[0], pk[1]);
        if (sub == 0) p.act_scales[((size_t)tile_m * p.act_blocks + k0 / 32) * 128 + fr] = f16_round_trip(dsc);
      }
    }
    }  // tile loop
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int NT, int EPI>
int32_t launch_nt(rmi_ctx* ctx, const gemm_params& p, size_t m_tiles) {
  constexpr size_t smem = 1024 + STAGES * stage_layout<NT>::BYTES + (EPI == GEMM_EPI_SWIGLU_Q8 ? 128 * 65 * 4 : 0);
  // SEM selects the accumulate (SCALAR: separate multiply and add; otherwise one fma per block) and the
  // quantizer of the SwiGLU epilogue.  AVX2 = the x86 quantizer with the whole-block fma chain; only the
  // SwiGLU epilogue quantizes, so the other epilogues share the NEON instantiation.
  auto kern = ctx->sem == RMI_SEM_SCALAR ? gemm_tc_kernel<NT, EPI, RMI_SEM_SCALAR>
              : (ctx->sem == RMI_SEM_AVX2 && EPI == GEMM_EPI_SWIGLU_Q8) ? gemm_tc_kernel<NT, EPI, RMI_SEM_AVX2>
                                                                        : gemm_tc_kernel<NT, EPI, RMI_SEM_NEON>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed: %s", smem, cudaGetErrorString(e));
    return RMI_ERR_CUDA;
  }
  gemm_params pp = p;
  pp.n_tiles = m_tiles * p.n_tiles_n;
  size_t grid = pp.n_tiles < (size_t)ctx->sm_count ? pp.n_tiles : (size_t)ctx->sm_count;
  const int pr = rmi_prof_begin(ctx, EPI == GEMM_EPI_SWIGLU_Q8 ? "gemm_tc_swiglu" : "gemm_tc");
  const cudaError_t le = rmi_launch(ctx, kern, dim3((unsigned)grid), dim3(THREADS), smem, pp);
  rmi_prof_end(ctx, pr);
  if (le != cudaSuccess) {
    rmi_set_error("launch of gemm_tc failed: %s", cudaGetErrorString(le));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "gemm_tc");
}

}  // namespace

int32_t launch_gemm_tc(rmi_ctx* ctx, const gemm_tc_args& a) {
  const rmi_weight* w = a.w;
  const bool swiglu = a.epilogue == GEMM_EPI_SWIGLU_Q8;
  RMI_REQUIRE((swiglu ? w->d_umma_gu_q : w->d_umma_q) != nullptr, RMI_ERR_BAD_HANDLE,
              "tcgen05 weight layout was not built");
  if (a.swap_ab) {
    // small batches: the weight is the 128-row operand, the activation rows are the tile columns, so no
    // tensor-core or epilogue work is spent on padding rows; the result is stored transposed
    RMI_REQUIRE(a.epilogue == GEMM_EPI_F32 && a.col_begin == 0 && a.col_end == w->n_rows, RMI_ERR_UNSUPPORTED,
                "swapped-operand GEMM: f32 output of all weight rows only");
    RMI_REQUIRE(w->d_umma_q != nullptr, RMI_ERR_BAD_HANDLE, "tcgen05 weight layout was not built");
    if (a.m == 0 || w->n_rows == 0) return RMI_OK;
    gemm_params p = {};
    p.a_img = w->d_umma_q;
    p.a_scales = w->d_umma_s;
    p.b_img = a.a_img;
    p.b_scales = a.a_scales;
    p.m = w->n_rows;
    p.n_rows_w = a.m;
    p.blocks = w->n_in / 32;
    p.n_slabs = (w->n_in + 127) / 128;
    p.col_begin = 0;
    p.col_end = a.m;
    p.out = a.out;
    p.out_stride = a.out_stride;
    p.status = ctx->d_status;
    p.fo = ctx->fanout;
    p.transpose = 1;
    p.n_tiles_n = (a.m + 31) / 32;
    return launch_nt<32, GEMM_EPI_F32>(ctx, p, (w->n_rows + 127) / 128);
  }
  gemm_params p = {};
  p.a_img = a.a_img;
  p.a_scales = a.a_scales;
  p.b_img = swiglu ? w->d_umma_gu_q : w->d_umma_q;
  p.b_scales = swiglu ? w->d_umma_gu_s : w->d_umma_s;
  p.m = a.m;
  p.n_rows_w = w->n_rows;
  p.blocks = w->n_in / 32;
  p.n_slabs = (w->n_in + 127) / 128;
  p.col_begin = a.col_begin;
  p.col_end = a.col_end;
  p.out = a.out;
  p.out_stride = a.out_stride;
  p.n_ff = a.n_ff;
  p.act_img = a.act_img;
  p.act_scales = a.act_scales;
  p.act_f32 = a.act_f32;
  p.sums = a.sums;
  p.status = ctx->d_status;
  p.fo = ctx->fanout;
  const size_t m_tiles = (a.m + 127) / 128;
  const size_t n_cols = a.col_end - a.col_begin;
  if (a.m == 0 || n_cols == 0) return RMI_OK;
  if (swiglu) {
    // col range is given in FFN columns; a tile of 64 interleaved weight rows covers 32 of them
    RMI_REQUIRE(a.n_ff % 32 == 0 && a.col_begin % 64 == 0 && n_cols % 32 == 0, RMI_ERR_BAD_SHAPE,
                "fused SwiGLU GEMM needs n_ff and the column range to be multiples of 32 (start: 64)");
    p.col_begin = a.col_begin * 2;
    p.col_end = a.col_end * 2;
    p.n_tiles_n = n_cols / 32;
    p.act_slabs = (a.n_ff + 127) / 128;
    p.act_blocks = a.n_ff / 32;
    return launch_nt<64, GEMM_EPI_SWIGLU_Q8>(ctx, p, m_tiles);
  }
  RMI_REQUIRE(a.col_begin % 128 == 0, RMI_ERR_BAD_SHAPE, "column range must start on a multiple of 128");
  // 64-column tiles unless that leaves SMs without work
  int nt = 64;
  if (m_tiles * ((n_cols + nt - 1) / nt) < 2 * (size_t)ctx->sm_count) nt = 32;
  p.n_tiles_n = (n_cols + nt - 1) / nt;
  if (a.epilogue == GEMM_EPI_BLOCK_SUMS) {
    if (nt == 64) return launch_nt<64, GEMM_EPI_BLOCK_SUMS>(ctx, p, m_tiles);
    return launch_nt<32, GEMM_EPI_BLOCK_SUMS>(ctx, p, m_tiles);
  }
  if (nt == 64) return launch_nt<64, GEMM_EPI_F32>(ctx, p, m_tiles);
  return launch_nt<32, GEMM_EPI_F32>(ctx, p, m_tiles);
}
