// Q8_0 x Q8_0 prefill GEMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// out[m, n] = sum over 32-blocks b of  f16(w.d[n,b]) * xs[m,b] * (int32 dot of block b)
// accumulated in block order exactly as the reference's whole-block variants do:
//   NEON    sum = fma(f32(dot), wd*xs, sum)     src/ops/kernel/q8_0/neon.rs:59-70
//   SCALAR  sum += (wd*xs) * f32(dot)           src/ops/kernel/q8_0/scalar.rs:42-56
//
// tcgen05.mma.kind::i8 has K = 32 per instruction = one Q8_0 block, so every MMA writes a
// fresh 128 x NT int32 tile into one of NBUF tensor-memory buffers and the epilogue warps
// drain it (tcgen05.ld), rescale and accumulate in f32 registers while the next MMAs run.
//
// Roles (320 threads): warp 0 = bulk-copy producer (cp.async.bulk into a 4-stage ring of
// 128-byte K slabs), warp 1 = TMEM owner + single-thread MMA issuer, warps 2..9 = epilogue
// (warp w may touch TMEM lanes 32*(w%4).., two warps per lane quadrant split the columns).
//
// Operands arrive pre-tiled in HBM in the tcgen05 K-major no-swizzle core-matrix order
// (8 rows x 16 B, LBO = 128 B along K, SBO = 1024 B along rows), so a stage is filled by
// contiguous bulk copies and no tensor map is needed.
//
// Every wait is bounded: after two seconds of failed polls a role records a site id in the
// context's status word, raises a shared abort flag that all other waits observe, and the
// CTA falls through to the common teardown (TMEM is always deallocated).
#include "common.cuh"
#include "kernels.cuh"

namespace {

constexpr int STAGES = 4;
constexpr int SLAB_BYTES_A = 128 * 128;  // 128 rows x 128 B of K
constexpr int NBUF = 4;
constexpr uint32_t WAIT_LIMIT = 1u << 26;
constexpr uint64_t WAIT_NS = 2000000000ull;  // 2 s

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
  size_t act_slabs, act_blocks;
  rmi_dev_status* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: gives up after WAIT_NS of wall time (or WAIT_LIMIT polls).  Returns false when
// the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          rmi_dev_status* status, int site, int detail) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255) {
      if (*abort_flag) return false;
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_NS) break;
    }
  }
  *abort_flag = 1;
  if (atomicCAS(&status->code, 0, RMI_ERR_TIMEOUT) == 0) {
    status->where = site;
    status->detail = detail;
  }
  return false;
}

__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
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

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
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

struct __align__(128) smem_layout_hdr {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tfull[NBUF];
  uint64_t tempty[NBUF];
  uint32_t tmem_base;
  int abort_flag;
};

// NT: tile columns (32, 64, 128).  EPI: GEMM_EPI_*.  SEM: RMI_SEM_NEON or RMI_SEM_SCALAR.
template <int NT, int EPI, int SEM>
__global__ void __launch_bounds__(320, 1) gemm_tc_kernel(const gemm_params p) {
  constexpr int CPW = NT / 2;              // columns per epilogue warp
  constexpr int B_STAGE = NT * 128;        // bytes of B per stage
  constexpr uint32_t TMEM_COLS = NBUF * NT < 32 ? 32 : NBUF * NT;  // 128, 256 or 512 (powers of two)
  extern __shared__ __align__(128) uint8_t smem_raw[];
  smem_layout_hdr* hdr = reinterpret_cast<smem_layout_hdr*>(smem_raw);
  uint8_t* stage_a = smem_raw + 1024;
  uint8_t* stage_b = stage_a + STAGES * SLAB_BYTES_A;
  volatile int* abort_flag = &hdr->abort_flag;

  const int warp = threadIdx.x / 32, lane = threadIdx.x & 31;
  const size_t tile_n = blockIdx.x % p.n_tiles_n, tile_m = blockIdx.x / p.n_tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; i++) {
      mbar_init(&hdr->full[i], 1);
      mbar_init(&hdr->empty[i], 1);
    }
    for (int i = 0; i < NBUF; i++) {
      mbar_init(&hdr->tfull[i], 1);
      mbar_init(&hdr->tempty[i], 8);
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

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      for (size_t s = 0; s < p.n_slabs; s++) {
        const int st = (int)(s % STAGES);
        const uint32_t ph = (uint32_t)((s / STAGES) & 1);
        if (s >= STAGES && !mbar_wait(&hdr->empty[st], ph ^ 1, abort_flag, p.status, 1, (int)s)) break;
        mbar_expect_tx(&hdr->full[st], SLAB_BYTES_A + B_STAGE);
        bulk_g2s(stage_a + st * SLAB_BYTES_A, p.a_img + (tile_m * p.n_slabs + s) * SLAB_BYTES_A, SLAB_BYTES_A,
                 &hdr->full[st]);
        uint8_t* bdst = stage_b + st * B_STAGE;
        if (EPI == GEMM_EPI_SWIGLU_Q8) {
          // rows: gate[j0..+31], up[j0..+31], gate[j0+32..+63], up[j0+32..+63]
          const size_t j0 = p.col_begin + tile_n * 64;
#pragma unroll
          for (int piece = 0; piece < 4; piece++) {
            const size_t wr = (piece & 1 ? p.n_ff : 0) + j0 + (piece >> 1) * 32;  // weight row
            const uint8_t* src = p.b_img + ((wr / 128) * p.n_slabs + s) * SLAB_BYTES_A + ((wr % 128) / 8) * 1024;
            bulk_g2s(bdst + piece * 4096, src, 4096, &hdr->full[st]);
          }
        } else {
          const size_t wr = p.col_begin + tile_n * NT;
          const uint8_t* src = p.b_img + ((wr / 128) * p.n_slabs + s) * SLAB_BYTES_A + ((wr % 128) / 8) * 1024;
          bulk_g2s(bdst, src, B_STAGE, &hdr->full[st]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8<NT>();
      size_t g = 0;
      bool ok = true;
      for (size_t s = 0; s < p.n_slabs && ok; s++) {
        const int st = (int)(s % STAGES);
        if (!mbar_wait(&hdr->full[st], (uint32_t)((s / STAGES) & 1), abort_flag, p.status, 2, (int)s)) break;
        tc_fence_after();
        const uint32_t a0 = smem_u32(stage_a + st * SLAB_BYTES_A), b0 = smem_u32(stage_b + st * B_STAGE);
        const size_t kb_n = p.blocks - s * 4 < 4 ? p.blocks - s * 4 : 4;
        for (size_t kb = 0; kb < kb_n; kb++, g++) {
          const int buf = (int)(g % NBUF);
          if (g >= NBUF && !mbar_wait(&hdr->tempty[buf], (uint32_t)(((g / NBUF) & 1) ^ 1), abort_flag, p.status, 3, (int)g)) {
            ok = false;
            break;
          }
          tc_fence_after();
          umma_i8(tmem_base + (uint32_t)(buf * NT), umma_desc(a0 + (uint32_t)kb * 256u),
                  umma_desc(b0 + (uint32_t)kb * 256u), idesc);
          umma_commit(&hdr->tfull[buf]);
        }
        umma_commit(&hdr->empty[st]);  // smem stage is free once these MMAs have read it
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps)
    const int q = warp % 4;                // TMEM lane quadrant this warp may access
    const int h = (warp - 2) / 4;          // which half of the tile columns
    const int r_tile = q * 32 + lane;      // row inside the 128-row tile
    const size_t row = tile_m * 128 + r_tile;
    float acc[CPW];
#pragma unroll
    for (int c = 0; c < CPW; c++) acc[c] = 0.0f;

    // weight-scale base pointers: scales are [tile128][block][128 rows]
    size_t wrow0, wrow1 = 0;  // first weight row of this warp's columns (second: up half)
    if (EPI == GEMM_EPI_SWIGLU_Q8) {
      wrow0 = p.col_begin + tile_n * 64 + h * 32;
      wrow1 = p.n_ff + wrow0;
    } else {
      wrow0 = p.col_begin + tile_n * NT + h * CPW;
    }
    const float* ws0 = p.b_scales ? p.b_scales + (wrow0 / 128) * p.blocks * 128 + (wrow0 % 128) : nullptr;
    const float* ws1 = p.b_scales ? p.b_scales + (wrow1 / 128) * p.blocks * 128 + (wrow1 % 128) : nullptr;
    const float* xsp = p.a_scales ? p.a_scales + tile_m * p.blocks * 128 + r_tile : nullptr;

    bool ok = true;
    for (size_t g = 0; g < p.blocks && ok; g++) {
      const int buf = (int)(g % NBUF);
      float xs = 0.0f;
      if (EPI != GEMM_EPI_BLOCK_SUMS) xs = __ldg(xsp + g * 128);
      if (!mbar_wait(&hdr->tfull[buf], (uint32_t)((g / NBUF) & 1), abort_flag, p.status, 4, (int)g)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * NT + h * CPW);
#pragma unroll
      for (int c0 = 0; c0 < CPW; c0 += 16) {
        int d[16];
        tmem_ld16(taddr + c0, d);
        tmem_ld_wait();
        if (c0 + 16 == CPW) {
          // all TMEM reads of this buffer are complete: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->tempty[buf]);
        }
        if (EPI == GEMM_EPI_BLOCK_SUMS) {
          if (row < p.m) {
#pragma unroll
            for (int c = 0; c < 16; c++) {
              size_t n = wrow0 + c0 + c;
              if (n < p.col_end) p.sums[(row * p.n_rows_w + n) * p.blocks + g] = d[c];
            }
          }
        } else {
          const float* wsp = (EPI == GEMM_EPI_SWIGLU_Q8 && c0 >= 32) ? ws1 + g * 128 + (c0 - 32) : ws0 + g * 128 + c0;
#pragma unroll
          for (int c4 = 0; c4 < 16; c4 += 4) {
            const float4 wd4 = __ldg(reinterpret_cast<const float4*>(wsp + c4));
            const float wdv[4] = {wd4.x, wd4.y, wd4.z, wd4.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const float s = __fmul_rn(wdv[j], xs);
              const float f = small_int_to_f32(d[c4 + j]);
              if (SEM == RMI_SEM_SCALAR) {
                acc[c0 + c4 + j] = __fadd_rn(acc[c0 + c4 + j], __fmul_rn(s, f));
              } else {
                acc[c0 + c4 + j] = __fmaf_rn(f, s, acc[c0 + c4 + j]);
              }
            }
          }
        }
      }
    }

    if (ok) {
      if (EPI == GEMM_EPI_F32) {
        if (row < p.m) {
          float* o = p.out + row * p.out_stride + wrow0;
          if (wrow0 + CPW <= p.col_end && ((p.out_stride | wrow0) & 3) == 0) {
#pragma unroll
            for (int c = 0; c < CPW; c += 4)
              *reinterpret_cast<float4*>(o + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
          } else {
#pragma unroll
            for (int c = 0; c < CPW; c++)
              if (wrow0 + c < p.col_end) o[c] = acc[c];
          }
        }
      } else if (EPI == GEMM_EPI_SWIGLU_Q8) {
        // src/ops/activation/mod.rs:137-151 then src/ops/quant/q8_0.rs (NEON / scalar form):
        // the 32 columns of this thread are exactly one Q8_0 block of the FFN activation.
        float v[32];
        float amax = 0.0f;
#pragma unroll
        for (int c = 0; c < 32; c++) {
          const float gte = acc[c % CPW], up = acc[(32 + c) % CPW];
          const float sl = __fdiv_rn(gte, __fadd_rn(1.0f, exp_cr(-gte)));
          v[c] = __fmul_rn(up, sl);
          amax = fmaxf(amax, fabsf(v[c]));
        }
        float dsc, inv;
        q8_scale_pair<SEM>(amax, &dsc, &inv);
        const size_t k0 = wrow0;  // column index inside n_ff
        if (p.act_f32 && row < p.m) {
#pragma unroll
          for (int c = 0; c < 32; c++) p.act_f32[row * p.n_ff + k0 + c] = v[c];
        }
        uint32_t packed[8];
#pragma unroll
        for (int w4 = 0; w4 < 8; w4++) {
          uint32_t u = 0;
#pragma unroll
          for (int j = 0; j < 4; j++) u |= (uint32_t)(uint8_t)(int8_t)q8_quant_value<SEM>(v[w4 * 4 + j], inv) << (8 * j);
          packed[w4] = u;
        }
        const size_t slab = k0 / 128, cc = (k0 % 128) / 16;
        uint8_t* img = p.act_img + (tile_m * p.act_slabs + slab) * SLAB_BYTES_A + (r_tile / 8) * 1024 + (r_tile % 8) * 16;
        *reinterpret_cast<uint4*>(img + cc * 128) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(img + (cc + 1) * 128) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        p.act_scales[(tile_m * p.act_blocks + k0 / 32) * 128 + r_tile] = f16_round_trip(dsc);
      }
    }
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
  constexpr size_t smem = 1024 + STAGES * (SLAB_BYTES_A + NT * 128);
  auto kern = ctx->sem == RMI_SEM_SCALAR ? gemm_tc_kernel<NT, EPI, RMI_SEM_SCALAR> : gemm_tc_kernel<NT, EPI, RMI_SEM_NEON>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed: %s", smem, cudaGetErrorString(e));
    return RMI_ERR_CUDA;
  }
  size_t grid = m_tiles * p.n_tiles_n;
  const int pr = rmi_prof_begin(ctx, EPI == GEMM_EPI_SWIGLU_Q8 ? "gemm_tc_swiglu" : "gemm_tc");
  kern<<<(unsigned)grid, 320, smem, ctx->stream>>>(p);
  rmi_prof_end(ctx, pr);
  return rmi_post_launch(ctx, "gemm_tc");
}

}  // namespace

int32_t launch_gemm_tc(rmi_ctx* ctx, const gemm_tc_args& a) {
  const rmi_weight* w = a.w;
  RMI_REQUIRE(w->d_umma_q != nullptr, RMI_ERR_BAD_HANDLE, "tcgen05 weight layout was not built");
  RMI_REQUIRE(ctx->sem != RMI_SEM_AVX2 || a.epilogue == GEMM_EPI_BLOCK_SUMS, RMI_ERR_UNSUPPORTED,
              "the tcgen05 GEMM accumulates whole-block sums (NEON or SCALAR semantics)");
  gemm_params p = {};
  p.a_img = a.a_img;
  p.a_scales = a.a_scales;
  p.b_img = w->d_umma_q;
  p.b_scales = w->d_umma_s;
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
  const size_t m_tiles = (a.m + 127) / 128;
  const size_t n_cols = a.col_end - a.col_begin;
  if (a.m == 0 || n_cols == 0) return RMI_OK;
  if (a.epilogue == GEMM_EPI_SWIGLU_Q8) {
    RMI_REQUIRE(a.n_ff % 64 == 0 && a.col_begin % 64 == 0 && n_cols % 64 == 0, RMI_ERR_BAD_SHAPE,
                "fused SwiGLU GEMM needs n_ff and the column range to be multiples of 64");
    p.n_tiles_n = n_cols / 64;
    p.act_slabs = (a.n_ff + 127) / 128;
    p.act_blocks = a.n_ff / 32;
    return launch_nt<128, GEMM_EPI_SWIGLU_Q8>(ctx, p, m_tiles);
  }
  RMI_REQUIRE(a.col_begin % 128 == 0, RMI_ERR_BAD_SHAPE, "column range must start on a multiple of 128");
  // largest tile width that still gives every SM a tile
  int nt = 128;
  while (nt > 32 && m_tiles * ((n_cols + nt - 1) / nt) < (size_t)ctx->sm_count) nt >>= 1;
  p.n_tiles_n = (n_cols + nt - 1) / nt;
  if (a.epilogue == GEMM_EPI_BLOCK_SUMS) {
    switch (nt) {
      case 128: return launch_nt<128, GEMM_EPI_BLOCK_SUMS>(ctx, p, m_tiles);
      case 64: return launch_nt<64, GEMM_EPI_BLOCK_SUMS>(ctx, p, m_tiles);
      default: return launch_nt<32, GEMM_EPI_BLOCK_SUMS>(ctx, p, m_tiles);
    }
  }
  switch (nt) {
    case 128: return launch_nt<128, GEMM_EPI_F32>(ctx, p, m_tiles);
    case 64: return launch_nt<64, GEMM_EPI_F32>(ctx, p, m_tiles);
    default: return launch_nt<32, GEMM_EPI_F32>(ctx, p, m_tiles);
  }
}
