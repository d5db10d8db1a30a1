// The banded prefill kernel (tcgen05), warp-specialised.  Included by prefill.cu after the PTX wrappers,
// descriptors, shared-memory plan and QuadPlan.
//
// One CTA (640 threads, one per SM) owns 256 query rows of one Q head: two 128-row MMA tiles X = 0, 1,
// each made of two 64-row query blocks, so every K / V tile that is fetched feeds four query blocks.
//   warp 0        producer: TMA copies of Q (once) and of the K / V blobs of every step, three stages ahead
//   warp 1        issuer:   all tcgen05.mma of the CTA (one elected thread)
//   warps 2-3     widen the INT8 V codes of a step to fp16 in shared memory (the P.V operand)
//   warps 4-19    softmax: tile X = (warp-4)/8, two threads per query row; warp w reads TMEM lanes
//                 32*(w%4)..+31, warps w and w+4 of a tile share 32 rows and split the 64 key columns and
//                 the 128 output channels in halves
//
// Per step (one 64-key tile) and MMA tile:
//   S[128x64]  = Q8 . K8^T            4 x kind::i8 (M128 N64 K32), s32 accumulators (bit-equal to the reference's)
//   P codes    = the reference's u8 quantisation of 2^(score - base) per row and tile (prefill_sm80.cu:386-414)
//   O[128x128] += (code * s) . V      4 x kind::f16 (M128 N128 K16): the per-tile scale s = 2^(base - ref) / 255 is
//                                     folded into the fp16 P operand, V codes are exact in fp16, and the fp32
//                                     accumulator stays in TMEM for the whole CTA
// where ref is a per-row reference exponent that is only moved (and O rescaled in TMEM) when a tile's
// maximum exceeds it by more than 2^8.  The reference instead reads an integer P.V accumulator out per
// tile and folds it into registers; both evaluate sum_t s_t * (codes_t . V) / sum_t s_t * sum(codes_t),
// here with one extra fp16 rounding (2^-12 relative) of each weight, far inside the output tolerance.
// Sink and diagonal tiles use fp16 weights and the fp16 V blob exactly like the reference.
//
// Every wait is an mbarrier wait with a time limit and the CTA-wide abort flag; there is no bar.sync
// between the initial and the final __syncthreads, so a role that gives up cannot strand another.
#pragma once
// (included inside namespace tri)

struct PrefillBarriers {
  uint64_t q;               // Q tiles landed
  uint64_t kv_full[3];      // K + raw V of a stage landed (transaction bytes)
  uint64_t kv_empty[3];     // stage reusable: QK^T done (tcgen05.commit) + both widening warps done
  uint64_t v16_full[2];     // fp16 V operand ready: two widening warps, or TMA of the fp16 blob + one plain arrive
  uint64_t v16_empty[2];    // all P.V of the step done
  uint64_t s_full[2][2];    // [tile][buffer] scores in TMEM
  uint64_t p_full[2][2];    // [tile][buffer] P operand written by the 8 softmax warps of the tile
  uint64_t o_done[2][2];    // [tile][buffer] P.V of that P buffer done
  uint64_t pair[2][4];      // [tile][lane quadrant] the two warps that share 32 rows exchanged their partial maxima
};

__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// grid = quads * batch * heads_q CTAs, heaviest query rows first; 640 threads; one CTA per SM.
template <typename Out>
__global__ void __launch_bounds__(PrefillThreads, 1) prefill_kernel(const __grid_constant__ CUtensorMap map_q8,
    const __grid_constant__ CUtensorMap map_q4, const int32_t* bands, const uint8_t* k8, const uint8_t* k4x, const float* ka8,
    const float* ka4, const uint8_t* v16, const uint8_t* v8, const float* qa8, const float* qa4, const float* vstat, Out* out,
    int64_t osb, int64_t osh, int64_t ost, int heads_q, int heads_kv, int tokens, int units_q, float sm_log2, int* err) {
  extern __shared__ uint8_t raw_smem[];
  __shared__ __align__(8) PrefillBarriers bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float xchg[2][2][2][128];   // [tile][parity][column half][row]: partial maxima, at the end denominators
  uint8_t* smem = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int rows = (tokens + BM - 1) / BM, quads = (rows + 3) / 4, tiles = rows;
  const int quad_id = quads - 1 - blockIdx.x / units_q, qunit = blockIdx.x % units_q;
  const int b = qunit / heads_q, h = qunit % heads_q, g = heads_q / heads_kv;
  const int64_t kvunit = (int64_t)b * heads_kv + h / g;
  const int w8 = bands[h * 2], w4 = bands[h * 2 + 1];
  if (w8 < 1) return;   // head handled elsewhere (un-quantised BF16 extension); uniform for the CTA
  QuadPlan plan;
  plan.build(quad_id, rows, w8, w4);
  const int nsteps = plan.steps();
  const bool need_q4 = plan.n4 > 0;

  // the visiting order as tables: tile | mode << 12, and the 4-bit mask of query blocks that take part
  uint16_t* step_tm = reinterpret_cast<uint16_t*>(smem + SmSteps);
  uint8_t* step_mask = smem + SmSteps + 2 * MaxSteps;
  for (int i = tid; i < nsteps; i += PrefillThreads) {
    int tile, mode, mask;
    plan.get(i, tile, mode, mask);
    step_tm[i] = (uint16_t)(tile | (mode << 12));
    step_mask[i] = (uint8_t)mask;
  }
  if (tid == 0) {
    mbar_init(&bars.q, 1);
    for (int s = 0; s < 3; ++s) { mbar_init(&bars.kv_full[s], 1); mbar_init(&bars.kv_empty[s], 3); }
    for (int s = 0; s < 2; ++s) { mbar_init(&bars.v16_full[s], 2); mbar_init(&bars.v16_empty[s], 1); }
    for (int x = 0; x < 2; ++x) {
      for (int s = 0; s < 2; ++s) { mbar_init(&bars.s_full[x][s], 1); mbar_init(&bars.p_full[x][s], 8); mbar_init(&bars.o_done[x][s], 1); }
      for (int qd = 0; qd < 4; ++qd) mbar_init(&bars.pair[x][qd], 2);
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
  auto wait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait_abortable(bar, parity & 1u, abortp); };

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(&bars.q, need_q4 ? 65536u : 32768u);
      for (int x = 0; x < 2; ++x) {
        tma_load_3d(smem + SmQ8 + x * 16384, &map_q8, 0, plan.q0 * BM + x * 128, qunit, &bars.q);
        if (need_q4) tma_load_3d(smem + SmQ4 + x * 16384, &map_q4, 0, plan.q0 * BM + x * 128, qunit, &bars.q);
      }
      for (int i = 0; i < nsteps; ++i) {
        const int tile = tile_of(i), mode = mode_of(i), s = i % 3, vb = i & 1;
        if (i >= 3 && !wait(&bars.kv_empty[s], i / 3 - 1)) break;
        const int64_t ht = kvunit * tiles + tile;
        if (mode == ModeF16) {
          if (i >= 2 && !wait(&bars.v16_empty[vb], (i - 2) >> 1)) break;
          mbar_expect_tx(&bars.kv_full[s], K8Bytes);
          bulk_g2s(smem + SmK + s * K8Bytes, k8 + ht * K8Bytes, K8Bytes, &bars.kv_full[s]);
          mbar_expect_tx(&bars.v16_full[vb], V16Bytes);   // first arrival; the second one follows the copy's issue
          bulk_g2s(smem + SmV16 + vb * V16Bytes, v16 + ht * V16Bytes, V16Bytes, &bars.v16_full[vb]);
          mbar_arrive_cta(&bars.v16_full[vb]);
        } else {
          mbar_expect_tx(&bars.kv_full[s], K8Bytes + V8Bytes);
          bulk_g2s(smem + SmK + s * K8Bytes, (mode == ModeQ4 ? k4x : k8) + ht * K8Bytes, K8Bytes, &bars.kv_full[s]);
          bulk_g2s(smem + SmV8 + s * V8Bytes, v8 + ht * V8Bytes, V8Bytes, &bars.kv_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- issuer -----------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t q8_addr = smem_u32(smem + SmQ8), q4_addr = smem_u32(smem + SmQ4);
      int nqk[2] = {0, 0}, npv[2] = {0, 0};
      auto issue_qk = [&](int i) -> bool {
        const int mode = mode_of(i), mask = step_mask[i], s = i % 3;
        if (!wait(&bars.kv_full[s], i / 3)) return false;
        tc_fence_after();
        const uint32_t ka_ = smem_u32(smem + SmK + s * K8Bytes);
        for (int x = 0; x < 2; ++x) {
          if (((mask >> (2 * x)) & 3) == 0) continue;
          const int sb = nqk[x] & 1;
          const uint32_t qa_ = (mode == ModeQ4 ? q4_addr : q8_addr) + x * 16384;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_i8(tmem + TmemS + x * 128 + sb * 64, smem_desc(qa_ + kk * 32, 0, 1024, Layout128B),
                    smem_desc(ka_ + kk * 256, 128, 1024, LayoutNone), IdescQK, kk > 0);
          tc_commit(&bars.s_full[x][sb]);
          ++nqk[x];
        }
        tc_commit(&bars.kv_empty[s]);
        return true;
      };
      bool ok = wait(&bars.q, 0) && issue_qk(0);
      for (int i = 0; ok && i < nsteps; ++i) {
        if (i + 1 < nsteps && !issue_qk(i + 1)) break;   // the next scores are computed while this step's softmax runs
        const int mask = step_mask[i], vb = i & 1;
        if (!wait(&bars.v16_full[vb], i >> 1)) break;
        const uint32_t va = smem_u32(smem + SmV16 + vb * V16Bytes);
        for (int x = 0; x < 2 && ok; ++x) {
          if (((mask >> (2 * x)) & 3) == 0) continue;
          const int pb = npv[x] & 1;
          if (!wait(&bars.p_full[x][pb], npv[x] >> 1)) { ok = false; break; }
          tc_fence_after();
          const uint32_t pa = smem_u32(smem + SmP + (2 * x + pb) * 16384);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem + TmemO + x * 128, smem_desc(pa + kk * 256, 128, 1024, LayoutNone),
                     smem_desc(va + kk * 256, 128, 1024, LayoutNone), IdescPV16, (npv[x] > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&bars.o_done[x][pb]);
          ++npv[x];
        }
        tc_commit(&bars.v16_empty[vb]);
      }
    }
  } else if (warp < 4) {
    // ---- V widening: int8 codes of the raw V stage -> fp16 operand ----------------------------------
    // A 16-byte unit of the V8 blob (one channel, 16 key positions) becomes two 16-byte units of the
    // fp16 operand (8 key positions each) in the same position order, which is the order the softmax
    // warps write P in.  Code c is built as the fp16 number 1024 + (c ^ 0x80) by byte shuffles; the
    // subtraction of 1152 is exact.
    const int ct = tid - 64;   // 0..63
    const __half2 bias = __half2half2(__float2half(1152.f));
    for (int i = 0; i < nsteps; ++i) {
      const int mode = mode_of(i), s = i % 3, vb = i & 1;
      if (!wait(&bars.kv_full[s], i / 3)) break;
      if (mode != ModeF16) {
        if (i >= 2 && !wait(&bars.v16_empty[vb], (i - 2) >> 1)) break;
        const uint4* src = reinterpret_cast<const uint4*>(smem + SmV8 + s * V8Bytes);
        uint8_t* dst = smem + SmV16 + vb * V16Bytes;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int unit = ct + 64 * u;                 // [ch/8][key/16][ch%8]
          const int cg = unit >> 5, run = (unit >> 3) & 3, r8 = unit & 7;
          const uint4 raw = src[unit];
          const uint32_t in[4] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u, raw.z ^ 0x80808080u, raw.w ^ 0x80808080u};
          uint32_t o[8];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t lo = __byte_perm(in[k], 0x64646464u, 0x4140), hi = __byte_perm(in[k], 0x64646464u, 0x4342);
            const __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias);
            const __half2 c = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
            o[2 * k] = *reinterpret_cast<const uint32_t*>(&a);
            o[2 * k + 1] = *reinterpret_cast<const uint32_t*>(&c);
          }
          uint8_t* d = dst + cg * 1024 + (2 * run) * 128 + r8 * 16;
          *reinterpret_cast<uint4*>(d) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(d + 128) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) {
        if (mode != ModeF16) mbar_arrive_cta(&bars.v16_full[vb]);
        mbar_arrive_cta(&bars.kv_empty[s]);
      }
    }
  } else {
    // ---- softmax ------------------------------------------------------------------------------------
    const int sw = warp - 4, x = sw / 8, quad = sw % 4, ch = (sw % 8) / 4;
    const int row = quad * 32 + lane, half = row / 64, blk = 2 * x + half;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    const int bh = plan.q0 + blk, qi = bh * BM + (row & 63);
    const bool row_valid = blk < plan.nb && qi < tokens;
    const int64_t qrow = (int64_t)qunit * tokens + qi;
    const float qs8 = row_valid ? qa8[qrow] * sm_log2 : FLT_MIN;
    const float qs4 = (row_valid && need_q4) ? qa4[qrow] * sm_log2 : FLT_MIN;
    float ref = -FLT_MAX, denom = 0.f;   // reference exponent of the row; this thread's share of the denominator
    int n = 0;                           // steps of this tile so far
    bool zero_rows[2] = {false, false};  // this thread's rows of P buffer [.] are known to be zero
    auto load_kscale = [&](int i) {
      return __ldg(reinterpret_cast<const float4*>((mode_of(i) == ModeQ4 ? ka4 : ka8) + (kvunit * tiles + tile_of(i)) * 4));
    };
    int inext = 0;   // next step in which this tile takes part
    while (inext < nsteps && ((step_mask[inext] >> (2 * x)) & 3) == 0) ++inext;
    float4 ks_next = inext < nsteps ? load_kscale(inext) : make_float4(0.f, 0.f, 0.f, 0.f);
    bool ok = true;
    while (inext < nsteps) {
      const int i = inext;
      const int tile = tile_of(i), mode = mode_of(i), mx = (step_mask[i] >> (2 * x)) & 3;
      const float ks[4] = {ks_next.x, ks_next.y, ks_next.z, ks_next.w};
      ++inext;
      while (inext < nsteps && ((step_mask[inext] >> (2 * x)) & 3) == 0) ++inext;
      if (inext < nsteps) ks_next = load_kscale(inext);   // in flight while this step computes
      const int sb = n & 1;
      if (!(ok = wait(&bars.s_full[x][sb], n >> 1))) break;
      tc_fence_after();
      const bool active = (mx >> half) & 1;   // uniform per warp
      const bool diag = mode == ModeF16 && tile == bh;
      const float qs = mode == ModeQ4 ? qs4 : qs8;
      const float slope[2] = {qs * ks[2 * ch], qs * ks[2 * ch + 1]};   // this thread's two 16-key groups
      const int key0 = tile * BN + 32 * ch;
      const uint32_t s_addr = lane_base + TmemS + x * 128 + sb * 64 + 32 * ch;
      auto dead = [&](int key) { return key >= tokens || key > qi || qi >= tokens; };   // diagonal tile only

      // pass 1: partial scaled maximum over this thread's 32 columns (prefill_sm80.cu:244-253)
      float part = -CUDART_INF_F;
      if (active) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t a[16];
          tmem_ld16(s_addr + 16 * cc, a);
          tmem_ld_wait();
          int mxi = INT_MIN;
          if (diag) {
#pragma unroll
            for (int j = 0; j < 16; ++j) if (!dead(key0 + 16 * cc + j)) mxi = max(mxi, (int)a[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) mxi = max(mxi, (int)a[j]);
          }
          if (mxi != INT_MIN) part = fmaxf(part, slope[cc] * (float)mxi);
        }
      }
      xchg[x][n & 1][ch][row] = part;
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(&bars.pair[x][quad]);
      if (!(ok = wait(&bars.pair[x][quad], n))) break;
      const float tmax = fmaxf(xchg[x][n & 1][0][row], xchg[x][n & 1][1][row]);

      // move the row's reference exponent when this tile towers over it, and rescale what O holds
      const bool move = active && tmax > ref + RefSlack;
      float factor = 1.f;
      if (move) {
        factor = ref > -FLT_MAX ? exp2f(ref - tmax) : 0.f;
        ref = tmax;
        denom *= factor;
      }
      if (n > 0 && __any_sync(0xffffffffu, move)) {
        if (!(ok = wait(&bars.o_done[x][(n - 1) & 1], (n - 1) >> 1))) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t a[16];
          const uint32_t o_addr = lane_base + TmemO + x * 128 + 64 * ch + 16 * c;
          tmem_ld16(o_addr, a);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) a[j] = __float_as_uint(__uint_as_float(a[j]) * factor);
          tmem_st16(o_addr, a);
        }
        tmem_st_wait();
      }
      if (n >= 2 && !(ok = wait(&bars.o_done[x][sb], (n - 2) >> 1))) break;   // P buffer sb is free again

      uint8_t* prow = smem + SmP + (2 * x + sb) * 16384 + (row / 8) * 1024 + (row % 8) * 16;   // core matrices [row/8][key/8]
      if (!active) {
        if (!zero_rows[sb]) {
#pragma unroll
          for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(prow + (4 * ch + c) * 128) = make_uint4(0u, 0u, 0u, 0u);
          zero_rows[sb] = true;
        }
      } else if (mode == ModeF16) {
        zero_rows[sb] = false;
        float sum = 0.f;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t a[16];
          tmem_ld16(s_addr + 16 * cc, a);
          tmem_ld_wait();
          const float off = fmaf(-slope[cc], 12582912.f, PShift - ref);
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            float e[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              e[u] = exp2f(fmaf(slope[cc], __int_as_float((int)a[j + u] + Magic), off));
              if (diag && dead(key0 + 16 * cc + j + u)) e[u] = 0.f;
            }
            const __half2 hp = __floats2half2_rn(e[0], e[1]);
            sum += __low2float(hp) + __high2float(hp);
            w[j / 2] = *reinterpret_cast<const uint32_t*>(&hp);
          }
          *reinterpret_cast<uint4*>(prow + (4 * ch + 2 * cc) * 128) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(prow + (4 * ch + 2 * cc + 1) * 128) = make_uint4(w[4], w[5], w[6], w[7]);
        }
        denom += sum;
      } else {
        // prefill_sm80.cu:386-414: u8 codes of 2^(score - base); band tiles are never masked
        zero_rows[sb] = false;
        const float ks_max = fmaxf(fmaxf(ks[0], ks[1]), fmaxf(ks[2], ks[3]));
        float base = tmax;
        base += tile_base_margin(qs * ks_max, base);
        // weight of one code step, rounded to fp16 once: numerator (tensor core) and denominator use the same value
        const __half sh = __float2half_rn(exp2f(base - ref + PShift) * (1.f / 255.f));
        const __half2 s2 = __half2half2(sh), nb2 = __half2half2(__hneg(__hmul(sh, __float2half(1024.f))));
        int rs = 0;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t a[16];
          tmem_ld16(s_addr + 16 * cc, a);
          tmem_ld_wait();
          uint32_t w[16];
          if (mode == ModeQ4) {
            // (float)acc without the conversion unit: exact for |acc| < 2^22
#pragma unroll
            for (int j = 0; j < 16; ++j)
              w[j] = __float_as_uint(fmaf(exp2f(fmaf(slope[cc], __int_as_float((int)a[j] + Magic) - 12582912.f, -base)), 255.f, PMagicHalf));
          } else {
            const float off = fmaf(-slope[cc], 12582912.f, -base);
#pragma unroll
            for (int j = 0; j < 16; ++j)
              w[j] = __float_as_uint(fmaf(exp2f(fmaf(slope[cc], __int_as_float((int)a[j] + Magic), off)), 255.f, PMagicHalf));
          }
          uint32_t hw[8];
#pragma unroll
          for (int sidx = 0; sidx < 4; ++sidx) {   // positions 4s..4s+3 of the run hold keys kperm(s, 0..3), like the V8 blob
            const uint32_t pw = pack_bytes(w[2 * sidx], w[2 * sidx + 1], w[2 * sidx + 8], w[2 * sidx + 9]);
            rs = (int)__dp4a(pw, 0x01010101u, (uint32_t)rs);
            const uint32_t lo = __byte_perm(pw, 0x64646464u, 0x4140), hi = __byte_perm(pw, 0x64646464u, 0x4342);
            const __half2 pl = __hfma2(*reinterpret_cast<const __half2*>(&lo), s2, nb2);   // (1024 + code) * s - 1024 * s
            const __half2 ph = __hfma2(*reinterpret_cast<const __half2*>(&hi), s2, nb2);
            hw[2 * sidx] = *reinterpret_cast<const uint32_t*>(&pl);
            hw[2 * sidx + 1] = *reinterpret_cast<const uint32_t*>(&ph);
          }
          *reinterpret_cast<uint4*>(prow + (4 * ch + 2 * cc) * 128) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
          *reinterpret_cast<uint4*>(prow + (4 * ch + 2 * cc + 1) * 128) = make_uint4(hw[4], hw[5], hw[6], hw[7]);
        }
        denom = fmaf((float)rs, __half2float(sh), denom);
      }
      fence_proxy_async_smem();   // P (generic-proxy stores) must be visible to the tensor core's async proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(&bars.p_full[x][sb]);
      ++n;
    }

    // ---- epilogue: O / denominator, de-normalised (prefill_sm80.cu:466-487) ----------------------------
    if (ok && n > 0) ok = wait(&bars.o_done[x][(n - 1) & 1], (n - 1) >> 1);
    if (ok && n > 0) {
      tc_fence_after();
      xchg[x][n & 1][ch][row] = denom;
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(&bars.pair[x][quad]);
      ok = wait(&bars.pair[x][quad], n);
    }
    if (ok && n > 0) {
      const float total = xchg[x][n & 1][0][row] + xchg[x][n & 1][1][row];
      const float inv = total > 0.f ? 1.f / total : 0.f;
      const float* mean = vstat + kvunit * StatFloats + 64 * ch;
      const float* scale = mean + D;
      Out* dst = out + b * osb + h * osh + (int64_t)qi * ost + 64 * ch;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t a[16];
        tmem_ld16(lane_base + TmemO + x * 128 + 64 * ch + 16 * c, a);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int v = 0; v < 2; ++v) {
            Out vals[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              vals[j] = to_out<Out>(fmaf(__uint_as_float(a[8 * v + j]) * inv, __ldg(scale + 16 * c + 8 * v + j), __ldg(mean + 16 * c + 8 * v + j)));
            *reinterpret_cast<uint4*>(dst + 16 * c + 8 * v) = *reinterpret_cast<const uint4*>(vals);
          }
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  const bool failed = *abortp != 0;
  if (failed) {   // a wait ran out: give copies / MMAs that may still be in flight a bounded time before the CTA goes away
    if (tid == 0) atomicExch(err, ErrBarrierTimeout);
    const uint64_t t_abort = globaltimer_ns();
    while (globaltimer_ns() - t_abort < 2000000ull) {}
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem, TmemCols);
}
