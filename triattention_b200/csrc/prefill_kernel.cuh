// The banded prefill kernel (tcgen05).  Included by prefill.cu after the PTX wrappers, descriptors,
// shared-memory plan and StepPlan.
//
// Thread layout: 256 threads, two per query row.  Warp w reads TMEM lanes 32*(w%4) .. +31 (the hardware
// ties a warp to that lane quadrant), so warps w and w+4 share 32 rows: warp w takes the first 32 key
// columns of the score tile and the first 64 output channels, warp w+4 the second halves.  Row state
// (running maximum, correction) is replicated in both threads of a row; the only exchange per tile is the
// row's partial maximum through shared memory.  Halving the per-thread work keeps the kernel at 128
// registers, so two CTAs (16 warps) are resident per SM and the ALU/MUFU-bound softmax has warps to
// overlap with the tensor core.
//
// Tensor-core schedule per step (thread 0 issues): P.V of step i, then QK^T of step i+1 right behind it,
// so the next scores are ready while this step's accumulators are folded into the registers.
#pragma once
// (included inside namespace tri)

// grid = pairs * batch * heads_q CTAs, heaviest query-block pairs first; 256 threads; 2 CTAs per SM.
template <typename Out>
__global__ void __launch_bounds__(PrefillThreads, 2) prefill_kernel(const __grid_constant__ CUtensorMap map_q8,
    const __grid_constant__ CUtensorMap map_q4, const int32_t* bands, const uint8_t* k8, const uint8_t* k4x, const float* ka8,
    const float* ka4, const uint8_t* v16, const uint8_t* v8, const float* qa8, const float* qa4, const float* vstat, Out* out,
    int64_t osb, int64_t osh, int64_t ost, int heads_q, int heads_kv, int tokens, int units_q, float sm_log2, int* err) {
  extern __shared__ uint8_t raw_smem[];
  __shared__ __align__(8) uint64_t bar_q, bar_kv[2], bar_s, bar_d;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float xchg[2][128];   // per-row partial maxima (and, at the end, denominators) of the two column halves
  uint8_t* smem = raw_smem + ((1024u - (smem_u32(raw_smem) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int quad = warp % 4, ch = warp / 4, row = quad * 32 + lane, half = row / 64;
  const int rows = (tokens + BM - 1) / BM, pairs = (rows + 1) / 2, tiles = rows;
  const int pair = pairs - 1 - blockIdx.x / units_q, qunit = blockIdx.x % units_q;
  const int b = qunit / heads_q, h = qunit % heads_q, g = heads_q / heads_kv;
  const int64_t kvunit = (int64_t)b * heads_kv + h / g;
  const int w8 = bands[h * 2], w4 = bands[h * 2 + 1];
  if (w8 < 1) return;   // head handled elsewhere (un-quantised BF16 extension); uniform for the CTA
  StepPlan plan;
  plan.build(pair, rows, w8, w4);
  const int nsteps = plan.steps();
  const bool need_q4 = plan.n4 > 0;

  // the visiting order as a table: tile | mode << 12 | half mask << 14
  uint16_t* steps = reinterpret_cast<uint16_t*>(smem + SmSteps);
  for (int i = tid; i < nsteps; i += PrefillThreads) {
    int tile, mode, mask;
    plan.get(i, tile, mode, mask);
    steps[i] = (uint16_t)(tile | (mode << 12) | (mask << 14));
  }
  auto step_tile = [&](int i) { return (int)(steps[i] & 0xfffu); };
  auto step_mode = [&](int i) { return (int)((steps[i] >> 12) & 3u); };
  auto step_mask = [&](int i) { return (int)(steps[i] >> 14); };
  if (tid == 0) {
    mbar_init(&bar_q, 1); mbar_init(&bar_kv[0], 1); mbar_init(&bar_kv[1], 1); mbar_init(&bar_s, 1); mbar_init(&bar_d, 1);
    mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, TmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  volatile int* abortp = &abort_flag;
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
  const uint32_t q8_addr = smem_u32(smem + SmQ8), q4_addr = smem_u32(smem + SmQ4), p_addr = smem_u32(smem + SmP);

  auto issue_loads = [&](int i) {   // thread 0 only
    const int tile = step_tile(i), mode = step_mode(i);
    const int s = i & 1;
    const int64_t ht = kvunit * tiles + tile;
    const uint32_t vbytes = mode == ModeF16 ? V16Bytes : V8Bytes;
    mbar_expect_tx(&bar_kv[s], K8Bytes + vbytes);
    bulk_g2s(smem + SmK + s * K8Bytes, (mode == ModeQ4 ? k4x : k8) + ht * K8Bytes, K8Bytes, &bar_kv[s]);
    bulk_g2s(smem + SmV + s * V16Bytes, mode == ModeF16 ? v16 + ht * V16Bytes : v8 + ht * V8Bytes, vbytes, &bar_kv[s]);
  };
  auto issue_qk = [&](int i) {      // thread 0 only: S = Q . K^T of step i, commit to bar_s
    const int tile = step_tile(i), mode = step_mode(i);
    const int s = i & 1;
    if (!mbar_wait_abortable(&bar_kv[s], (i >> 1) & 1, abortp)) return;
    tc_fence_after();
    const uint32_t qa_ = mode == ModeQ4 ? q4_addr : q8_addr, ka_ = smem_u32(smem + SmK + s * K8Bytes);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      umma_i8(tmem + TmemS, smem_desc(qa_ + kk * 32, 0, 1024, Layout128B), smem_desc(ka_ + kk * 256, 128, 1024, LayoutNone),
              IdescQK, kk > 0);
    tc_commit(&bar_s);
  };
  if (tid == 0) {
    mbar_expect_tx(&bar_q, need_q4 ? 32768u : 16384u);
    tma_load_3d(smem + SmQ8, &map_q8, 0, plan.b0 * BM, qunit, &bar_q);
    if (need_q4) tma_load_3d(smem + SmQ4, &map_q4, 0, plan.b0 * BM, qunit, &bar_q);
    issue_loads(0);
    if (mbar_wait_abortable(&bar_q, 0, abortp)) issue_qk(0);
  }

  // per-row state; this thread owns columns 32*ch .. +31 of the scores and channels 64*ch .. +63 of the output
  const int bh = plan.b0 + half, qi = bh * BM + (row & 63);
  const bool row_valid = (half == 0 || plan.has1) && qi < tokens;
  const int64_t qrow = (int64_t)qunit * tokens + qi;
  const float qs8 = row_valid ? qa8[qrow] * sm_log2 : FLT_MIN;
  const float qs4 = (row_valid && need_q4) ? qa4[qrow] * sm_log2 : FLT_MIN;
  float o[64];
#pragma unroll
  for (int j = 0; j < 64; ++j) o[j] = 0.f;
  float m = -FLT_MAX, denom = 0.f, corr = 0.f;   // denom: this thread's share of the row's denominator
  int n8seen = 0;
  uint32_t ph_s = 0, ph_d = 0;
  uint8_t* prow8 = smem + SmP + (row / 8) * 512 + (row % 8) * 16;     // u8 P row: core matrices [row/8][key/16]
  uint8_t* prow16 = smem + SmP + (row / 8) * 1024 + (row % 8) * 16;   // fp16 P row: core matrices [row/8][key/8]

  auto load_kscale = [&](int i) {   // the four K scales of step i's tile (16-byte aligned)
    const int tile = step_tile(i), mode = step_mode(i);
    return __ldg(reinterpret_cast<const float4*>((mode == ModeQ4 ? ka4 : ka8) + (kvunit * tiles + tile) * 4));
  };
  float4 ks_next = load_kscale(0);
  // o += D * factor for this thread's 64 channels; integer accumulators are read through the 2^23+2^22 bias
  // like the reference's (prefill_sm80.cu:420), fp32 ones (FP16-PV tiles) directly
  auto read_accumulators = [&](bool f16, float factor) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t a[16];
      tmem_ld16(lane_base + TmemD + 64 * ch + 16 * c, a);
      tmem_ld_wait();
      if (f16) {
#pragma unroll
        for (int j = 0; j < 16; ++j) o[c * 16 + j] = fmaf(__uint_as_float(a[j]), factor, o[c * 16 + j]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) o[c * 16 + j] = fmaf(__int_as_float((int)a[j] + Magic), factor, o[c * 16 + j]);
      }
    }
  };
  bool pend = false, pend_act = false, pend_f16 = false;   // a P.V whose accumulators have not been read yet
  float pend_bq = 0.f;

  for (int i = 0; i < nsteps; ++i) {
    const int tile = step_tile(i), mode = step_mode(i), mask = step_mask(i);
    const int s = i & 1;
    if (tid == 0 && i + 1 < nsteps) issue_loads(i + 1);   // stage (i+1)&1 was released by step i-1
    const bool have_s = mbar_wait_abortable(&bar_s, ph_s, abortp);
    ph_s ^= 1;
    tc_fence_after();
    const bool active = have_s && ((mask >> half) & 1);
    const bool diag = tile == bh;
    const float qs = mode == ModeQ4 ? qs4 : qs8;
    const float ks[4] = {ks_next.x, ks_next.y, ks_next.z, ks_next.w};
    if (i + 1 < nsteps) ks_next = load_kscale(i + 1);   // in flight while this step computes
    const float slope[2] = {qs * ks[2 * ch], qs * ks[2 * ch + 1]};   // this thread's two 16-key groups
    const int key0 = tile * BN + 32 * ch;
    auto dead = [&](int key) { return key >= tokens || key > qi || qi >= tokens; };   // diagonal tile only

    // pass 1: partial scaled maximum over this thread's 32 columns (prefill_sm80.cu:244-253)
    if (active) {
      float part = -CUDART_INF_F;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t a[16];
        tmem_ld16(lane_base + TmemS + 32 * ch + 16 * cc, a);
        tmem_ld_wait();
        int mx = INT_MIN;
        if (diag) {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (!dead(key0 + 16 * cc + j)) mx = max(mx, (int)a[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) mx = max(mx, (int)a[j]);
        }
        if (mx != INT_MIN) part = fmaxf(part, slope[cc] * (float)mx);
      }
      xchg[ch][row] = part;
    }
    __syncthreads();
    float bq = 0.f, alpha_i = 1.f, tmax = -CUDART_INF_F;
    if (active) {
      tmax = fmaxf(xchg[0][row], xchg[1][row]);
      const float n = fmaxf(m, tmax), alpha = exp2f(m - n);
      m = n;
      alpha_i = alpha;
      bool flush = false;
      if (mode != ModeF16) { flush = (n8seen % 16) == 15; ++n8seen; }
      if (flush || alpha != 1.f) {   // prefill_sm80.cu:350-357
        const float shift = -corr * alpha;
#pragma unroll
        for (int j = 0; j < 64; ++j) o[j] = fmaf(o[j], alpha, shift);
        corr = 0.f;
      }
    }
    // The previous step's P.V has had this step's first pass to finish; P may only be overwritten once it
    // is done.  Its accumulators are read further down, after this step's exponentials.
    bool have_d = true;
    if (pend) {
      have_d = mbar_wait_abortable(&bar_d, ph_d, abortp);
      ph_d ^= 1;
      tc_fence_after();
    }
    if (active) {
      const float alpha = alpha_i;
      if (mode == ModeF16) {
        denom *= alpha;
        float sum = 0.f;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t a[16];
          tmem_ld16(lane_base + TmemS + 32 * ch + 16 * cc, a);
          tmem_ld_wait();
          const float off = fmaf(-slope[cc], 12582912.f, -m);
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
          *reinterpret_cast<uint4*>(prow16 + (4 * ch + 2 * cc) * 128) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(prow16 + (4 * ch + 2 * cc + 1) * 128) = make_uint4(w[4], w[5], w[6], w[7]);
        }
        denom += sum;
      } else {
        // prefill_sm80.cu:386-414; band tiles are never masked
        const float ks_max = fmaxf(fmaxf(ks[0], ks[1]), fmaxf(ks[2], ks[3]));
        float base = tmax > -CUDART_INF_F ? tmax : m;
        base += tile_base_margin(qs * ks_max, base);
        bq = exp2f(base - m) / 255.f;
        int rs = 0;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t a[16];
          tmem_ld16(lane_base + TmemS + 32 * ch + 16 * cc, a);
          tmem_ld_wait();
          const float off = mode == ModeQ4 ? -base : fmaf(-slope[cc], 12582912.f, -base);
          uint32_t w[16];
          if (mode == ModeQ4) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              w[j] = __float_as_uint(fmaf(exp2f(fmaf(slope[cc], (float)(int)a[j], off)), 255.f, PMagicHalf));
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              w[j] = __float_as_uint(fmaf(exp2f(fmaf(slope[cc], __int_as_float((int)a[j] + Magic), off)), 255.f, PMagicHalf));
          }
          uint32_t pw[4];
#pragma unroll
          for (int sidx = 0; sidx < 4; ++sidx) {   // byte 4s+b of the run holds key kperm(s,b), like the V8 blob
            pw[sidx] = pack_bytes(w[2 * sidx], w[2 * sidx + 1], w[2 * sidx + 8], w[2 * sidx + 9]);
            rs = (int)__dp4a(pw[sidx], 0x01010101u, (uint32_t)rs);
          }
          *reinterpret_cast<uint4*>(prow8 + (2 * ch + cc) * 128) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        }
        denom = fmaf((float)rs, bq, denom * alpha);
        corr = fmaf(12582912.f, bq, corr);
      }
    }
    // fold the previous step's accumulators in now (deferred so that its MMA latency is hidden behind this
    // step's softmax).  This row's running output was already rescaled by this step's alpha, so the late
    // contribution takes the same factor.
    if (pend && pend_act && have_d) read_accumulators(pend_f16, pend_f16 ? alpha_i : pend_bq * alpha_i);
    // rows of an idle half keep stale P bytes: each output row depends only on its own P row, and idle
    // rows never read their accumulators
    fence_proxy_async_smem();   // P (generic-proxy stores) must be visible to the tensor core's async proxy
    tc_fence_before();
    __syncthreads();            // P complete, S consumed
    if (tid == 0 && !*abortp) {
      tc_fence_after();
      const uint32_t va = smem_u32(smem + SmV + s * V16Bytes);
      if (mode == ModeF16) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_f16(tmem + TmemD, smem_desc(p_addr + kk * 256, 128, 1024, LayoutNone), smem_desc(va + kk * 256, 128, 1024, LayoutNone),
                   IdescPV16, kk > 0);
      } else {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
          umma_i8(tmem + TmemD, smem_desc(p_addr + kk * 256, 128, 512, LayoutNone), smem_desc(va + kk * 256, 128, 512, LayoutNone),
                  IdescPV8, kk > 0);
      }
      tc_commit(&bar_d);
      if (i + 1 < nsteps) issue_qk(i + 1);   // the next scores are computed while this step's accumulators are read
    }
    __syncwarp();
    pend = true; pend_act = active; pend_f16 = mode == ModeF16; pend_bq = bq;
    // No barrier here: the next step waits for bar_d before it touches P, and the accumulators D are only
    // overwritten by the next P.V, which is issued behind the next step's second barrier.
  }
  if (pend) {   // the last step's accumulators
    const bool have_d = mbar_wait_abortable(&bar_d, ph_d, abortp);
    tc_fence_after();
    if (pend_act && have_d) read_accumulators(pend_f16, pend_f16 ? 1.f : pend_bq);
  }

  // the row's denominator is the sum of the two column halves' shares
  xchg[ch][row] = denom;
  __syncthreads();
  const bool ok = !*abortp;
  if (!ok && tid == 0) atomicExch(err, ErrBarrierTimeout);
  if (ok && row_valid) {
    // prefill_sm80.cu:466-487
    const float total = xchg[0][row] + xchg[1][row];
    const float inv = total > 0.f ? 1.f / total : 0.f;
    const float* mean = vstat + kvunit * StatFloats + 64 * ch;
    const float* scale = mean + D;
    Out* dst = out + b * osb + h * osh + (int64_t)qi * ost + 64 * ch;
#pragma unroll
    for (int c = 0; c < 64; c += 8) {
      Out vals[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) vals[j] = to_out<Out>(fmaf((o[c + j] - corr) * inv, __ldg(scale + c + j), __ldg(mean + c + j)));
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(vals);
    }
  }
  if (!ok) {   // a wait ran out: give copies / MMAs that may still be in flight a bounded time before the CTA goes away
    const uint64_t t_abort = globaltimer_ns();
    while (globaltimer_ns() - t_abort < 2000000ull) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TmemCols);
}
