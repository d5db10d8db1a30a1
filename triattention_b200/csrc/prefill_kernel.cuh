// The banded prefill kernel (tcgen05), warp-specialised.  Included by prefill.cu after the PTX wrappers,
// descriptors, shared-memory plan and QuadPlan.
//
// One CTA (640 threads, one per SM) owns 256 query rows of one Q head: two 128-row MMA tiles X = 0, 1,
// each made of two 64-row query blocks, so every K / V tile that is fetched feeds four query blocks.
//   warp 0        producer: TMA copies of Q (once) and of the K / V blobs of every step (K four steps ahead, V two)
//   warps 1-2     issue the QK^T side of MMA tile 0 / 1: bias + INT8 MMAs of every step (one elected thread each)
//   warp 3        issues the P.V side of both tiles (one elected thread)
//   warps 4-19    softmax: tile X = (warp-4)/8, two threads per query row; warp w reads TMEM lanes
//                 32*(w%4)..+31 (the hardware ties a warp to that lane quadrant), warps w and w+4 of a tile
//                 share 32 rows and split the 64 key columns and the 128 output channels in halves; their
//                 only exchange per step is the row's partial maximum (shared memory + a 64-thread barrier).
//                 Four softmax warps per scheduler are what it takes to keep the exponential unit busy:
//                 one warp alone issues an ex2 every ~15 cycles, the unit takes one every ~8.
//
// Integer scores are read as floats without a conversion: before the INT8 MMAs of a step the issuer presets the
// score buffer to 0x4B400000 (the bits of 12582912.0f, the bias the reference adds in registers,
// prefill_sm80.cu:27) with one fp16 MMA of constant operands, the QK^T MMAs accumulate on top, and for
// |score| < 2^22 the result read as a float IS 12582912 + score.  Row maxima are taken on those floats with the
// three-input max.
//
// P never touches shared memory: a softmax thread writes its fp16 weights over its own 32 score columns
// (one tcgen05.st per 16-key group: the group's high parts over the first 8 of its 16 columns, its low parts over
// the last 8) once it has read them, and the P.V MMAs
// take their A operand from tensor memory.
// The bias MMA of two steps later overwrites P; its issuer waits for that P.V to have completed first.  With A in tensor memory an M128 N128 K16 MMA takes 65 cycles instead of 108 (measured).
//
// Per step (one 64-key tile) and MMA tile:
//   S[128x64]  = Q8 . K8^T            4 x kind::i8 (M128 N64 K32), s32 accumulators (bit-equal to the reference's)
//   P codes    = the reference's u8 quantisation of 2^(score - base) per row and tile (prefill_sm80.cu:386-414)
//   O[128x128] += (code * s) . V      8 x kind::f16 (M128 N128 K16): the per-tile scale s = 2^(base - ref) / 255 is
//                                     folded into the P operand, which goes in as two fp16 parts, high (exact) + low,
//                                     whose sum is code * s to 2^-15 (4 MMAs each over the same V operand); V codes are
//                                     exact in fp16, and the fp32 accumulator stays in TMEM for the whole CTA
// where ref is a per-row reference exponent that is only moved (and O rescaled in TMEM) when a tile's
// maximum exceeds it by more than 2^8.  The reference instead reads an integer P.V accumulator out per
// tile and folds it into registers; both evaluate sum_t s_t * (codes_t . V) / sum_t s_t * sum(codes_t) over the same
// integer-code products; the reference's float32 accumulator (biased by 12582912 per tile) is the noisier of the two.
// Sink and diagonal tiles use fp16 weights and the fp16 V blob exactly like the reference.
//
// Every mbarrier wait has a time limit and obeys the CTA-wide abort flag (a wait that runs out leaves its site in the
// flag, and the kernel reports it with the error word).  The only other barrier inside
// the main loop is the 64-thread bar.sync of a softmax warp pair; both warps of a pair walk the same step
// list and reach it the same number of times even after an abort (they then skip everything else).
#pragma once
// (included inside namespace tri)

struct PrefillBarriers {
  uint64_t q;               // Q tiles landed
  uint64_t k_full[4];       // K tile + its scales landed (transaction bytes)
  uint64_t k_empty[4];      // K stage reusable: QK^T of both tiles done (one tcgen05.commit per tile)
  uint64_t v16_full[2];     // fp16 V operand landed (fp16 V' blob of sink / diagonal tiles, fp16 code blob otherwise)
  uint64_t v16_empty[2];    // P.V of both tiles done
  uint64_t s_full[2][2];    // [tile][buffer] scores in TMEM
  uint64_t p_full[2][2];    // [tile][buffer] P written over the score buffer by the 8 softmax warps of the tile
  uint64_t o_done[2][2];    // [tile][buffer] P.V of that P buffer done
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// column (inside a score buffer) of the P words of key group kk: the first half of the columns of the thread that owns it
// column (inside a score buffer) of the P words of key group kk (16 keys = 8 columns of fp16 pairs): key groups 2c and 2c+1
// belong to the thread that owns score columns 32c .. 32c+31; a key group's high parts sit over the first 8 of its own 16
// score columns and its low parts over the last 8, so that the thread stores both with one 16-column tcgen05.st
__device__ __forceinline__ constexpr uint32_t p_column(int kk) { return (kk >> 1) * 32 + (kk & 1) * 16; }
constexpr uint32_t PLow = 8;
// Two fp32 fused multiply-adds in one instruction (fma.rn.ftz.f32x2): each lane rounds exactly like the scalar fma, so the
// results are bit-identical; it halves the issue slots of the two fmas every score costs.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.ftz.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void pair_sync(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// grid = quads * batch * heads_q CTAs, heaviest query rows first; 640 threads; one CTA per SM.
template <typename Out, bool Raw>
__global__ void __launch_bounds__(PrefillThreads, 1) prefill_kernel(const __grid_constant__ CUtensorMap map_q8,
    const __grid_constant__ CUtensorMap map_q4, const __grid_constant__ CUtensorMap map_qraw,
    const __grid_constant__ CUtensorMap map_kraw, int has_raw, const int32_t* bands, const uint8_t* k8, const uint8_t* k4x, const float* ka8,
    const float* ka4, const uint8_t* v16, const uint8_t* v8h, const float* qa8, const float* qa4, const float* vstat, Out* out,
    int64_t osb, int64_t osh, int64_t ost, int64_t osc, int heads_q, int heads_kv, int tokens, int units_q, float sm_log2, int* err) {
  extern __shared__ uint8_t raw_smem[];
  __shared__ __align__(8) PrefillBarriers bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float k_scales[8][4];   // ring: the four K scales of the tiles of the last 8 steps, fetched with the tile
  __shared__ int steps_of_tile[2];       // number of steps in which MMA tile x takes part
  __shared__ float xchg[2][2][2][128];   // [tile][parity][column half][row]: partial maxima, at the end denominators
  uint8_t* smem = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int rows = (tokens + BM - 1) / BM, quads = (rows + 3) / 4, tiles = rows;
  const int quad_id = quads - 1 - blockIdx.x / units_q, qunit = blockIdx.x % units_q;
  const int b = qunit / heads_q, h = qunit % heads_q, g = heads_q / heads_kv;
  const int64_t kvunit = (int64_t)b * heads_kv + h / g;
  // blockIdx.y = band configuration of a sweep (one launch evaluates several maps over the same operands; 0 otherwise):
  // its own [Hq,2] band table and its own output tensor.  gridDim.x may cover only the last query rows (heaviest first).
  bands += (int64_t)blockIdx.y * heads_q * 2;
  out += (int64_t)blockIdx.y * osc;
  const int w8 = bands[h * 2], w4 = bands[h * 2 + 1];
  // A head with w8 < 1 belongs to an un-quantised (BF16) KV group: exact attention over every causal tile, straight
  // from the raw bf16 Q and K rows (TMA tensor copies of the caller's tensors) and the fp16 V blobs.  Uniform for the CTA.
  // (two instantiations: Raw = false serves the quantised heads, Raw = true the un-quantised ones; a CTA of the other
  // kind leaves at once, so the arithmetic of one kind costs the other neither registers nor instructions)
  constexpr bool raw = Raw;
  if ((w8 < 1) != Raw || (Raw && !has_raw)) return;
  QuadPlan plan;
  plan.build(quad_id, rows, raw ? (1 << 20) : w8, raw ? (1 << 20) : w4);
  const int nsteps = plan.steps();
  const bool need_q4 = !raw && plan.n4 > 0;
  const int kmask = raw ? 1 : 3, kshift = raw ? 1 : 2;   // K ring: four 8 KB stages of codes, or two 16 KB stages of bf16 rows

  // the visiting order as tables: tile | mode << 12, and the 4-bit mask of query blocks that take part
  uint16_t* step_tm = reinterpret_cast<uint16_t*>(smem + SmSteps);
  uint8_t* step_mask = smem + SmSteps + 2 * MaxSteps;
  for (int i = tid; i < nsteps; i += PrefillThreads) {
    int tile, mode, mask;
    plan.get(i, tile, mode, mask);
    step_tm[i] = (uint16_t)(tile | (mode << 12));
    step_mask[i] = (uint8_t)mask;
  }
  // per MMA tile the steps in which it takes part, in order, one word each: step | tile << 13 | mode << 24 | block mask << 26
  // (warps 1 and 2 list tile 0 / 1, 32 steps per round)
  uint32_t* step_list = reinterpret_cast<uint32_t*>(smem + SmSteps + StepBytes);
  if (warp == 1 || warp == 2) {
    const int x = warp - 1;
    int count = 0;
    for (int c = 0; c < nsteps; c += 32) {
      int tile = 0, mode = 0, mask = 0;
      if (c + lane < nsteps) plan.get(c + lane, tile, mode, mask);
      const int mx = (mask >> (2 * x)) & 3;
      const uint32_t votes = __ballot_sync(0xffffffffu, mx != 0);
      if (mx != 0)
        step_list[x * MaxSteps + count + __popc(votes & ((1u << lane) - 1u))] =
            (uint32_t)(c + lane) | ((uint32_t)tile << 13) | ((uint32_t)mode << 24) | ((uint32_t)mx << 26);
      count += __popc(votes);
    }
    if (lane == 0) steps_of_tile[x] = count;
  }
  for (int i = tid; i < (4096 + 2048) / 4; i += PrefillThreads)   // 3072.0 (0x6A00) for A, 256.0 (0x5C00) for B
    reinterpret_cast<uint32_t*>(smem + SmBiasA)[i] = i < 1024 ? 0x6A006A00u : 0x5C005C00u;
  fence_proxy_async_smem();
  if (tid == 0) {
    mbar_init(&bars.q, 1);
    for (int s = 0; s < 4; ++s) { mbar_init(&bars.k_full[s], 1); mbar_init(&bars.k_empty[s], 2); }
    for (int s = 0; s < 2; ++s) { mbar_init(&bars.v16_full[s], 1); mbar_init(&bars.v16_empty[s], 1); }
    for (int x = 0; x < 2; ++x) {
      for (int s = 0; s < 2; ++s) { mbar_init(&bars.s_full[x][s], 1); mbar_init(&bars.p_full[x][s], 4 * RowSplit); mbar_init(&bars.o_done[x][s], 1); }
    }
    mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, TmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abortp = &abort_flag;
  const uint32_t tmem = tmem_slot;
  auto tile_of = [&](int i) { return (int)(step_tm[i] & 0xfffu); };
  auto mode_of = [&](int i) { return (int)(step_tm[i] >> 12); };
  // site: which wait this is (reported with the error word when it runs out): 1 Q, 2 K stage free, 3 V stage free, 4 K landed,
  // 5 score buffer free, 6 V landed, 7 / 8 P of tile 0 / 1, 9 scores, 11 O before a rescale, 12 last P.V; the softmax
  // sites add the tile's step number << 8
  auto wait = [&](uint64_t* bar, uint32_t parity, int site) { return mbar_wait_parked(bar, parity & 1u, abortp, site); };

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------------
    if (lane == 0) {
      if (raw) {
        // bf16 Q rows of the caller's tensor: per MMA tile two boxes of 128 rows x 64 features (128-byte swizzle)
        mbar_expect_tx(&bars.q, 65536u);
        for (int x = 0; x < 2; ++x)
          for (int half = 0; half < 2; ++half)
            tma_load_4d(smem + SmQ8 + x * 32768 + half * 16384, &map_qraw, half * 64, plan.q0 * BM + x * 128, h, b, &bars.q);
      } else {
        mbar_expect_tx(&bars.q, need_q4 ? 65536u : 32768u);
        for (int x = 0; x < 2; ++x) {
          tma_load_3d(smem + SmQ8 + x * 16384, &map_q8, 0, plan.q0 * BM + x * 128, qunit, &bars.q);
          if (need_q4) tma_load_3d(smem + SmQ4 + x * 16384, &map_q4, 0, plan.q0 * BM + x * 128, qunit, &bars.q);
        }
      }
      for (int i = 0; i < nsteps; ++i) {
        const int tile = tile_of(i), mode = mode_of(i), s = i & kmask, vb = i & 1;
        if (i > kmask && !wait(&bars.k_empty[s], (i >> kshift) - 1, 2)) break;
        const int64_t ht = kvunit * tiles + tile;
        if (raw) {
          // the tile's 64 bf16 K rows from the caller's tensor: two boxes of 64 keys x 64 features
          mbar_expect_tx(&bars.k_full[s], 2 * K8Bytes);
          for (int half = 0; half < 2; ++half)
            tma_load_4d(smem + SmK + s * 2 * K8Bytes + half * K8Bytes, &map_kraw, half * 64, tile * BN, h / g, b, &bars.k_full[s]);
        } else {
          mbar_expect_tx(&bars.k_full[s], K8Bytes + 16);
          bulk_g2s(smem + SmK + s * K8Bytes, (mode == ModeQ4 ? k4x : k8) + ht * K8Bytes, K8Bytes, &bars.k_full[s]);
          bulk_g2s(&k_scales[i & 7][0], (mode == ModeQ4 ? ka4 : ka8) + ht * 4, 16, &bars.k_full[s]);
        }
        // the fp16 P.V operand of the step: V' itself for sink / diagonal tiles (and for every tile of an un-quantised
        // head, whose V' is V), the INT8 codes as fp16 numbers otherwise
        if (i >= 2 && !wait(&bars.v16_empty[vb], (i - 2) >> 1, 3)) break;
        mbar_expect_tx(&bars.v16_full[vb], V16Bytes);
        bulk_g2s(smem + SmV16 + vb * V16Bytes, ((raw || mode == ModeF16) ? v16 : v8h) + ht * V16Bytes, V16Bytes, &bars.v16_full[vb]);
      }
    }
  } else if (warp < 3) {
    // ---- QK^T issuers: warp 1 for MMA tile 0, warp 2 for tile 1 ---------------------------------------------
    // Three threads issue MMAs (QK^T of tile 0, QK^T of tile 1, P.V): most of an issuing thread's time goes into its own dependent
    // scalar instructions and into blocking on the pipe's queue, so a single thread for all 18 MMAs of a step was
    // the critical path of the CTA.  The tensor pipe orders nothing between different issuing threads; what one
    // needs from another it waits for explicitly: the score buffer of step n is free once the P.V of the tile's
    // step n-2 (which read P out of it) has completed.
    if (lane == 0) {
      const int x = warp - 1;
      // Descriptors are built once; per MMA only the 16-byte-unit address field (low word) moves.
      auto at = [](uint64_t desc, uint32_t byte_offset) { return desc + (uint64_t)(byte_offset >> 4); };   // stays inside the 14-bit field
      const uint64_t dq8 = smem_desc(smem_u32(smem + SmQ8 + x * 16384), 0, 1024, Layout128B);
      const uint64_t dq4 = smem_desc(smem_u32(smem + SmQ4 + x * 16384), 0, 1024, Layout128B);
      const uint64_t dk = smem_desc(smem_u32(smem + SmK), 128, 1024, LayoutNone);
      const uint64_t dba = smem_desc(smem_u32(smem + SmBiasA), 128, 256, LayoutNone), dbb = smem_desc(smem_u32(smem + SmBiasB), 128, 256, LayoutNone);
      const uint32_t st = tmem + TmemS + x * 128;
      int nqk = 0;
      bool ok = wait(&bars.q, 0, 1);
      const uint64_t dqr = smem_desc(smem_u32(smem + SmQ8 + x * 32768), 0, 1024, Layout128B);   // bf16 rows, both 128-byte swizzled
      const uint64_t dkr = smem_desc(smem_u32(smem + SmK), 0, 1024, Layout128B);
      for (int i = 0; ok && i < nsteps; ++i) {
        const int s = i & kmask;
        // every step, also those this tile sits out: an issuer that ran a ring round ahead would arrive twice on the
        // same k_empty phase
        if (!(ok = wait(&bars.k_full[s], i >> kshift, 4))) break;
        if ((step_mask[i] >> (2 * x)) & 3) {
          const int sb = nqk & 1;
          if (nqk >= 2 && !(ok = wait(&bars.o_done[x][sb], (nqk - 2) >> 1, 5))) break;
          tc_fence_after();
          if (raw) {
            // S = Q . K^T on bf16 rows, fp32 accumulators: 8 MMAs of 16 features; feature half hf sits in its own box
            const uint64_t dks = at(dkr, s * 2 * K8Bytes);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_f16(st + sb * 64, at(dqr, (kk >> 2) * 16384 + (kk & 3) * 32), at(dks, (kk >> 2) * K8Bytes + (kk & 3) * 32),
                       IdescQKRaw, kk > 0 ? 1u : 0u);
          } else {
            const uint64_t dqm = mode_of(i) == ModeQ4 ? dq4 : dq8, dks = at(dk, s * K8Bytes);
            umma_f16(st + sb * 64, dba, dbb, IdescBias, 0u);   // the bias (and the end of the P that lived here)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_i8(st + sb * 64, at(dqm, kk * 32), at(dks, kk * 256), IdescQK, 1u);
          }
          tc_commit(&bars.s_full[x][sb]);
          ++nqk;
        }
        tc_commit(&bars.k_empty[s]);   // one arrival per tile and step, also for steps the tile sits out
      }
    }
  } else if (warp == 3) {
    // ---- P.V issuer (both tiles) ------------------------------------------------------------------------------
    if (lane == 0) {
      auto at = [](uint64_t desc, uint32_t byte_offset) { return desc + (uint64_t)(byte_offset >> 4); };
      const uint64_t dv = smem_desc(smem_u32(smem + SmV16), 128, 1024, LayoutNone);
      int npv0 = 0, npv1 = 0;
      bool ok = true;
      for (int i = 0; ok && i < nsteps; ++i) {
        const int mask = step_mask[i], vb = i & 1;
        const bool two_part = !raw && mode_of(i) != ModeF16;   // quantised weights come as high + low fp16 parts
        if (!(ok = wait(&bars.v16_full[vb], i >> 1, 6))) break;
        const uint64_t dvs = at(dv, vb * V16Bytes);
        if (mask & 3) {
          const int pb = npv0 & 1;
          if (!(ok = wait(&bars.p_full[0][pb], npv0 >> 1, 7))) break;
          tc_fence_after();
          // P: key group kk (16 keys = 8 columns of fp16 pairs) sits in the first half of the 32 score columns of the
          // thread that computed it: columns 0-15 (keys 0-31) and 32-47 (keys 32-63) of score buffer pb
          const uint32_t pt = tmem + TmemS + pb * 64;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ts(tmem + TmemO, pt + p_column(kk), at(dvs, kk * 256), IdescPV16, (npv0 > 0 || kk > 0) ? 1u : 0u);
          if (two_part) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_f16_ts(tmem + TmemO, pt + p_column(kk) + PLow, at(dvs, kk * 256), IdescPV16, 1u);
          }
          tc_commit(&bars.o_done[0][pb]);
          ++npv0;
        }
        if (mask & 12) {
          const int pb = npv1 & 1;
          if (!(ok = wait(&bars.p_full[1][pb], npv1 >> 1, 8))) break;
          tc_fence_after();
          const uint32_t pt = tmem + TmemS + 128 + pb * 64;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ts(tmem + TmemO + 128, pt + p_column(kk), at(dvs, kk * 256), IdescPV16, (npv1 > 0 || kk > 0) ? 1u : 0u);
          if (two_part) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_f16_ts(tmem + TmemO + 128, pt + p_column(kk) + PLow, at(dvs, kk * 256), IdescPV16, 1u);
          }
          tc_commit(&bars.o_done[1][pb]);
          ++npv1;
        }
        tc_commit(&bars.v16_empty[vb]);
      }
    }
  } else {
    // ---- softmax ------------------------------------------------------------------------------------
    constexpr int G = 4 / RowSplit;   // 16-key groups per thread
    const int sw = warp - 4, x = sw / (4 * RowSplit), quad = warp % 4, ch = (sw % (4 * RowSplit)) / 4;
    const int row = quad * 32 + lane, half = row / 64, blk = 2 * x + half;
    const int pair_id = 1 + 4 * x + quad;   // named barrier of the two warps that share these 32 rows
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    const int bh = plan.q0 + blk, qi = bh * BM + (row & 63);
    const bool row_valid = blk < plan.nb && qi < tokens;
    const int64_t qrow = (int64_t)qunit * tokens + qi;
    const float qs8 = (row_valid && !raw) ? qa8[qrow] * sm_log2 : FLT_MIN;
    const float qs4 = (row_valid && need_q4) ? qa4[qrow] * sm_log2 : FLT_MIN;
    float ref = -FLT_MAX, denom = 0.f;   // reference exponent of the row; this thread's share of the denominator
    const int nx = steps_of_tile[x];     // steps of this tile
    // No result of a wait is looked at here: after an abort (a wait that ran out anywhere in the CTA) every wait returns at
    // once and the warp runs through its remaining steps on whatever the tensor memory holds (its own columns, so nothing
    // is touched that is not this CTA's); the kernel reports the error and the host discards the output.
    for (int n = 0; n < nx; ++n) {
      const uint32_t entry = step_list[x * MaxSteps + n];
      const int i = entry & 0x1fff, tile = (entry >> 13) & 0x7ff, mode = (entry >> 24) & 3, mx = entry >> 26;
      const int sb = n & 1;
      const bool active = (mx >> half) & 1;   // uniform for the warp pair
      const bool diag = mode == ModeF16 && tile == bh;
      const float qs = mode == ModeQ4 ? qs4 : qs8;
      const int key0 = tile * BN + 16 * G * ch;
      const uint32_t s_addr = lane_base + TmemS + x * 128 + sb * 64 + 16 * G * ch;
      auto dead = [&](int key) { return key >= tokens || key > qi || qi >= tokens; };   // diagonal tile only
      // P goes over this thread's 32 score columns: two fp16 weights per column, keys in natural order like both fp16
      // V blobs (p_column)

      wait(&bars.s_full[x][sb], n >> 1, 9 | (n << 8));
      tc_fence_after();
      // The tile's K scales came with the tile (the ring slot is not reused before step i+8, and the producer
      // cannot be more than 4 steps ahead of a softmax warp).
      const float4 ks = raw ? make_float4(1.f, 1.f, 1.f, 1.f) : *reinterpret_cast<const float4*>(&k_scales[i & 7][0]);
      float slope[G];   // one per 16-key group of this thread
      if constexpr (RowSplit == 2) { slope[0] = qs * (ch ? ks.z : ks.x); slope[1] = qs * (ch ? ks.w : ks.y); }
      else { slope[0] = qs * ks.x; slope[1] = qs * ks.y; slope[G - 2] = qs * ks.z; slope[G - 1] = qs * ks.w; }
      if (raw) {
#pragma unroll
        for (int cc = 0; cc < G; ++cc) slope[cc] = sm_log2;   // scores are plain fp32 dot products
      }
      float tmax = -CUDART_INF_F;
      uint32_t a[G][16];   // this thread's scores as float bits (12582912 + score); read once per step
      if (active) {
        // partial scaled maximum over this thread's 32 columns (prefill_sm80.cu:244-253), then the row's
        float part = -CUDART_INF_F;
        {
          tmem_ld32(s_addr, reinterpret_cast<uint32_t(&)[32]>(a));
          tmem_ld_wait();
#pragma unroll
          for (int cc = 0; cc < G; ++cc) {
            if (raw) {   // plain fp32 scores (sm_log2 > 0, so the scaled maximum is the scaled maximum score)
              float m = -CUDART_INF_F;
#pragma unroll
              for (int j = 0; j < 16; ++j) if (!diag || !dead(key0 + 16 * cc + j)) m = fmaxf(m, __uint_as_float(a[cc][j]));
              part = fmaxf(part, sm_log2 * m);
              continue;
            }
            float m = 0.f;   // below every biased score
            if (diag) {
#pragma unroll
              for (int j = 0; j < 16; ++j) if (!dead(key0 + 16 * cc + j)) m = fmaxf(m, __uint_as_float(a[cc][j]));
            } else {
              m = __uint_as_float(a[cc][0]);
#pragma unroll
              for (int j = 1; j < 15; j += 2) m = fmax3(m, __uint_as_float(a[cc][j]), __uint_as_float(a[cc][j + 1]));
              m = fmaxf(m, __uint_as_float(a[cc][15]));
            }
            if (m > 0.f) part = fmaxf(part, slope[cc] * (m - 12582912.f));
          }
        }
        if constexpr (RowSplit == 2) {
          xchg[x][sb][ch][row] = part;
          pair_sync(pair_id);
          tmax = fmaxf(xchg[x][sb][0][row], xchg[x][sb][1][row]);
        } else {
          tmax = part;
        }
      }
      if (active) {
        // Move the row's reference exponent, and rescale what O holds, when this tile towers over it.  In the fp16
        // steps (sink and diagonal tiles, the first steps of a row, in the reference's order) it moves with every
        // increase, so that it IS the reference's running maximum m there: the reference rounds 2^(score - m) to fp16
        // (prefill_sm80.cu:362-373), and only the same exponent gives the same rounding.  That costs one rescale of a
        // one-tile accumulator per row.  In the quantised steps the codes do not depend on the running maximum.
        // In a quantised step the exponent that matters is the tile's base (its maximum plus the reference's margin):
        // the weight of one code step is 2^(base - ref) / 255, kept below 2^(RefSlack + PShift) / 255 so that 1024 times
        // it stays inside fp16.
        const bool quantised = !raw && mode != ModeF16;
        const float ks_top = fmaxf(fmaxf(ks.x, ks.y), fmaxf(ks.z, ks.w));
        const float top = quantised ? tmax + tile_base_margin(qs * ks_top, tmax) : tmax;
        const bool move = (mode == ModeF16 && !raw) ? top > ref : top > ref + RefSlack;
        float factor = 1.f;
        if (move) {
          factor = ref > -FLT_MAX ? exp2f(ref - top) : 0.f;
          ref = top;
          denom *= factor;
        }
        if (n > 0 && __any_sync(0xffffffffu, move)) {
          wait(&bars.o_done[x][(n - 1) & 1], (n - 1) >> 1, 11 | (n << 8));
          {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 2 * G; ++c) {
              uint32_t o[16];
              const uint32_t o_addr = lane_base + TmemO + x * 128 + 32 * G * ch + 16 * c;
              tmem_ld16(o_addr, o);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
              tmem_st16(o_addr, o);
            }
            tmem_ld32(s_addr, reinterpret_cast<uint32_t(&)[32]>(a));   // read again: the scores need not survive
            tmem_ld_wait();                                            // the (rare) rescale in registers
          }
        }
      }
      if (!active) {
        const uint32_t zero[16] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};   // this half's rows contribute nothing
#pragma unroll
        for (int cc = 0; cc < G; ++cc) tmem_st16(s_addr + 16 * cc, zero);   // high and low parts (the latter unread in fp16 mode)
      } else if (mode == ModeF16 || raw) {
        float sum = 0.f;
#pragma unroll
        for (int cc = 0; cc < G; ++cc) {
          // quantised heads: the reference's expression, bit for bit, then x 2^PShift (exact); plain scores carry no bias
          const float off = raw ? -ref : fmaf(-slope[cc], 12582912.f, -ref);
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            float e[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              e[u] = exp2f(fmaf(slope[cc], __uint_as_float(a[cc][j + u]), off)) * PScale;
              if (diag && dead(key0 + 16 * cc + j + u)) e[u] = 0.f;
            }
            const __half2 hp = __floats2half2_rn(e[0], e[1]);
            sum += __low2float(hp) + __high2float(hp);
            w[j / 2] = *reinterpret_cast<const uint32_t*>(&hp);
          }
          tmem_st8(s_addr + 16 * cc, w);
        }
        denom += sum;
      } else {
        // prefill_sm80.cu:386-414: u8 codes of 2^(score - base); band tiles are never masked
        const float ks_max = fmaxf(fmaxf(ks.x, ks.y), fmaxf(ks.z, ks.w));
        float base = tmax;
        base += tile_base_margin(qs * ks_max, base);
        // Weight of one code step, s = 2^(base - ref) / 255 (times 2^PShift), split as s_hi + s_lo: s_hi = s rounded to
        // 3 significant bits, so that code * s_hi (8 + 3 bits) is EXACT in fp16, and s_lo = fp16(s - s_hi), at most
        // 2^-3 of s.  Each weight goes to the tensor core as two fp16 operands, p_hi = code * s_hi (exact) and
        // p_lo = fp16(code * s_lo) (one rounding, 2^-12 of a part that is at most 2^-3 of the weight), so p_hi + p_lo =
        // code * s to 2^-15 at worst: the tensor core sums the integer-code products the reference sums per tile
        // (prefill_sm80.cu:416-449), scaled like its fp32 `bq`, to well below the float32 noise of the reference's own
        // accumulator.  (A single fp16 weight, 2^-12 relative, left outputs in x20 outlier channels of V up to 0.009
        // from the reference.)  The denominator uses the same s_hi + s_lo.
        const float sf = exp2f(base - ref + PShift) * (1.f / 255.f);
        const float sf_hi = __uint_as_float((__float_as_uint(sf) + 0x00100000u) & 0xffe00000u);
        // both parts, and -1024 times both, with two packing conversions (the conversion unit is the exponential unit's)
        const __half2 parts = __floats2half2_rn(sf_hi, sf - sf_hi);
        const __half2 shi2 = __low2half2(parts), slo2 = __high2half2(parts);
        const __half2 nparts = __hmul2(parts, __half2half2(__float2half(-1024.f)));   // exact: a power of two
        const __half2 nhi2 = __low2half2(nparts), nlo2 = __high2half2(nparts);
        const float s_sum = sf_hi + __high2float(parts);   // what the two operand parts add up to, for the denominator
        int rs = 0;
        // The code is byte 1 of fma(2^x, 255, 2^15 + ... + 0.5) exactly as in the reference (prefill_sm80.cu:78-88);
        // this constant of the same binade also leaves 0x64 in byte 2, so that bytes 1-2 of the word are the
        // fp16 number 1024 + code.  Eight keys at a time to keep the live registers low.  The INT4 pass takes
        // (float)acc (exact for |acc| < 2^22) and rounds once like the reference's conversion; the INT8 pass keeps
        // the bias inside the fma like the reference does.
        auto codes = [&](auto int4_pass) {
          constexpr bool Int4 = decltype(int4_pass)::value;
#pragma unroll
          for (int cc = 0; cc < G; ++cc) {
            const float off = Int4 ? -base : fmaf(-slope[cc], 12582912.f, -base);
            uint32_t hl[16];   // the 16 weights of this key group, two per word: high parts in words 0-7, low parts in 8-15
            uint32_t* const hi = hl;
            uint32_t* const lo = hl + 8;
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
              uint32_t w[8];
#pragma unroll
              for (int u = 0; u < 8; u += 2) {   // two scores per fused multiply-add
                const int j = 8 * hb + u;
                const float s0 = Int4 ? __uint_as_float(a[cc][j]) - 12582912.f : __uint_as_float(a[cc][j]);
                const float s1 = Int4 ? __uint_as_float(a[cc][j + 1]) - 12582912.f : __uint_as_float(a[cc][j + 1]);
                float x0, x1, y0, y1;
                ffma2(x0, x1, slope[cc], slope[cc], s0, s1, off, off);
                ffma2(y0, y1, exp2f(x0), exp2f(x1), 255.f, 255.f, PMagic64, PMagic64);
                w[u] = __float_as_uint(y0);
                w[u + 1] = __float_as_uint(y1);
              }
              const uint32_t h0 = __byte_perm(w[0], w[1], 0x6521), h1 = __byte_perm(w[2], w[3], 0x6521);   // (1024 + code) x 2 as fp16
              const uint32_t h2 = __byte_perm(w[4], w[5], 0x6521), h3 = __byte_perm(w[6], w[7], 0x6521);
              rs = (int)__dp4a(h0, 0x00010001u, (uint32_t)rs);   // sum of the codes
              rs = (int)__dp4a(h1, 0x00010001u, (uint32_t)rs);
              rs = (int)__dp4a(h2, 0x00010001u, (uint32_t)rs);
              rs = (int)__dp4a(h3, 0x00010001u, (uint32_t)rs);
              // (1024 + code) * s - 1024 * s in one fused operation: code * s rounded once (exact for s_hi)
              const __half2 p0 = __hfma2(*reinterpret_cast<const __half2*>(&h0), shi2, nhi2);
              const __half2 p1 = __hfma2(*reinterpret_cast<const __half2*>(&h1), shi2, nhi2);
              const __half2 p2 = __hfma2(*reinterpret_cast<const __half2*>(&h2), shi2, nhi2);
              const __half2 p3 = __hfma2(*reinterpret_cast<const __half2*>(&h3), shi2, nhi2);
              hi[4 * hb] = *reinterpret_cast<const uint32_t*>(&p0); hi[4 * hb + 1] = *reinterpret_cast<const uint32_t*>(&p1);
              hi[4 * hb + 2] = *reinterpret_cast<const uint32_t*>(&p2); hi[4 * hb + 3] = *reinterpret_cast<const uint32_t*>(&p3);
              const __half2 l0 = __hfma2(*reinterpret_cast<const __half2*>(&h0), slo2, nlo2);
              const __half2 l1 = __hfma2(*reinterpret_cast<const __half2*>(&h1), slo2, nlo2);
              const __half2 l2 = __hfma2(*reinterpret_cast<const __half2*>(&h2), slo2, nlo2);
              const __half2 l3 = __hfma2(*reinterpret_cast<const __half2*>(&h3), slo2, nlo2);
              lo[4 * hb] = *reinterpret_cast<const uint32_t*>(&l0); lo[4 * hb + 1] = *reinterpret_cast<const uint32_t*>(&l1);
              lo[4 * hb + 2] = *reinterpret_cast<const uint32_t*>(&l2); lo[4 * hb + 3] = *reinterpret_cast<const uint32_t*>(&l3);
            }
            tmem_st16(s_addr + 16 * cc, hl);   // one store per key group: its high parts, then its low parts
          }
        };
        if (mode == ModeQ4) codes(std::true_type{}); else codes(std::false_type{});
        denom = fmaf((float)rs, s_sum, denom);
      }
      tmem_st_wait();   // P is in tensor memory before the issuer is told
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(&bars.p_full[x][sb]);
    }

    // ---- epilogue: O / denominator, de-normalised (prefill_sm80.cu:466-487) ----------------------------
    if (nx > 0) {
      const int n = nx;
      wait(&bars.o_done[x][(n - 1) & 1], (n - 1) >> 1, 12 | (n << 8));
      if constexpr (RowSplit == 2) {
        xchg[x][n & 1][ch][row] = denom;
        pair_sync(pair_id);
      }
      {
        tc_fence_after();
        const float total = RowSplit == 2 ? xchg[x][n & 1][0][row] + xchg[x][n & 1][1][row] : denom;
        const float inv = total > 0.f ? 1.f / total : 0.f;
        const float* mean = vstat + kvunit * StatFloats + 32 * G * ch;
        const float* scale = mean + D;
        Out* dst = out + b * osb + h * osh + (int64_t)qi * ost + 32 * G * ch;
#pragma unroll
        for (int c = 0; c < 2 * G; ++c) {
          uint32_t o[16];
          tmem_ld16(lane_base + TmemO + x * 128 + 32 * G * ch + 16 * c, o);
          tmem_ld_wait();
          if (row_valid) {
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              Out vals[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                vals[j] = to_out<Out>(fmaf(__uint_as_float(o[8 * v + j]) * inv, __ldg(scale + 16 * c + 8 * v + j), __ldg(mean + 16 * c + 8 * v + j)));
              *reinterpret_cast<uint4*>(dst + 16 * c + 8 * v) = *reinterpret_cast<const uint4*>(vals);
            }
          }
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  const int failed = *abortp;
  if (failed) {   // a wait ran out: give copies / MMAs that may still be in flight a bounded time before the CTA goes away
    if (tid == 0) atomicExch(err, ErrBarrierTimeout | (failed << 8));   // upper bits: which wait (site, and the tile's step)
    const uint64_t t_abort = globaltimer_ns();
    while (globaltimer_ns() - t_abort < 2000000ull) {}
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem, TmemCols);
}
