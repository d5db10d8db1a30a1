// Split-KV decode kernel, sm_100a: persistent warp-specialised CTAs streaming an equal share of the
// cache bytes each.  Included by decode.cu.
//
// Replaces triattention/kernels/cuda/common_device.cuh:178-371 (decode_tile, decode_kernel) of the
// reference.  The arithmetic per tile is the reference's (same float expressions, same 8-bit / 4-bit
// P codes with the accumulator's low byte as dither); the organisation is not:
//   * one CTA per SM; the last warp is the producer: it walks the CTA's tile list and keeps a
//     12-stage shared-memory ring full with TMA bulk copies (one per tile chunk, mbarrier transaction
//     counts);
//   * the other ConsumerWarps warps are consumers.  Each owns whole tiles (tile t of the CTA goes to
//     warp t % ConsumerWarps), so the probabilities never leave registers: the accumulator fragment
//     of QK^T is repacked in place as the A fragment of P.V.  No block barrier and no shared-memory
//     exchange per tile;
//   * a CTA's tile list is a contiguous slice of the global tile sequence cut by cost, so all CTAs
//     finish together; where the slice crosses a (sequence, KV head) boundary the consumers fold
//     their states through shared memory and emit one partial (m, l, o) per segment.
// Tile chunk layouts in the cache pool (written by cache_store_kernel; a lane reads 16 contiguous
// bytes and a warp 512 contiguous bytes per load):
//   K8 [key/8][half][key%8][sub][16 B]   16 B = features 32*sub + 16*half + 0..15 of the key
//   K4 [key/8][key%8][sub][16 B]         word s, byte j: low nibble = feature 32*sub+8s+j, high = +4
//   V8 [ch/8][ch%8][sub][16 B]           word w, byte j: key 16w + kperm(sub, j)
//   V4 [ch/8][ch%8][sub][8 B]            word kc, byte j: low = key 32kc+kperm(sub,j), high = +16
//   BF16 K [key/8][u][key%8][sub][16 B]  16 B = features 32*sub + 8u + 0..7;  32 keys per chunk
//   BF16 V [ch/8][ch%8][sub][16 B]       word 2ks+h = keys 16ks + 8h + 2sub + {0,1} of the channel
// In every integer contraction the k index is only a position; Q fragments are gathered with the
// same feature permutation, P fragments come out of the accumulators in the V blobs' key order.
#pragma once
#include "common.cuh"

namespace tri {

constexpr int ConsumerWarps = 6;
constexpr int DecodeThreads = (ConsumerWarps + 1) * 32;
constexpr int DecodeStages = 12;
// A stage must always be consumed by the same warp: a consumer that could run a whole ring round ahead
// of another would see the stage's barrier parity of two phases ago and read stale bytes.
static_assert(DecodeStages % ConsumerWarps == 0, "stage ownership");
constexpr int StageBytes = 16512;                      // >= 8192 + 8192 + 16, multiple of 128
constexpr int Bf16ChunkKeys = 32, Bf16ChunkBytes = 16384;
constexpr int CombFloats = MaxGroup * D + 2 * MaxGroup;
// per-warp fold slot (CombFloats floats); its first 2 KB double as the warp's Q scratch between folds
constexpr int SmRing = 0, SmComb = DecodeStages * StageBytes;
constexpr int DecodeShared = SmComb + ConsumerWarps * CombFloats * 4;
static_assert(DecodeShared <= 227 * 1024 && CombFloats * 4 >= 2048, "decode shared-memory plan");

// tile_info bits
constexpr uint32_t InfoTileMask = 0xfffu, InfoRowShift = 12, InfoK4 = 1u << 20, InfoV4 = 1u << 21, InfoBf16 = 1u << 22;
// A tile appended after the prompt (generated keys folded into the cache) holds 64 live keys (32 for a BF16 chunk) wherever
// the prompt ended: it is not masked against the prompt length.
constexpr uint32_t InfoFull = 1u << 23;

__device__ __forceinline__ uint32_t chunk_bytes(uint32_t info) {
  if (info & InfoBf16) return Bf16ChunkBytes;
  return ((info & InfoK4) ? K4Bytes : K8Bytes) + ((info & InfoV4) ? V4Bytes : V8Bytes) + 16;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() {   // the consumer warps only
  asm volatile("bar.sync 1, %0;" ::"n"(ConsumerWarps * 32) : "memory");
}

struct WarpState {        // online-softmax state of one consumer warp; lane = (row = lane/4, sub = lane%4)
  float m, denom, corr;   // denom is the lane's share; the quad is summed when the segment ends
  float out[16][2];       // channels 8*cb + 2*sub + {0,1}
};

// One quantised 64-key tile, whole warp.  common_device.cuh:178-273 of the reference, per row.
template <bool K4, bool V4>
__device__ __forceinline__ void quantised_tile(const uint8_t* stage, const uint32_t (&qf)[4][2], float qs, WarpState& st,
    int key_begin, int prompt, bool row_on) {
  const int lane = threadIdx.x % 32, group = lane / 4, sub = lane % 4;
  constexpr int KB = K4 ? K4Bytes : K8Bytes, VB = V4 ? V4Bytes : V8Bytes;
  const uint8_t* vb = stage + KB;
  const float4 kt4 = *reinterpret_cast<const float4*>(stage + KB + VB);
  const float kt[4] = {kt4.x, kt4.y, kt4.z, kt4.w};
  int c[8][4];
#pragma unroll
  for (int nb = 0; nb < 8; ++nb) {
    c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0;
    if constexpr (!K4) {
      const uint4 u0 = *reinterpret_cast<const uint4*>(stage + nb * 1024 + group * 64 + sub * 16);
      const uint4 u1 = *reinterpret_cast<const uint4*>(stage + nb * 1024 + 512 + group * 64 + sub * 16);
      mma_s8(c[nb], qf[0][0], qf[0][1], u0.x, u0.y);
      mma_s8(c[nb], qf[1][0], qf[1][1], u0.z, u0.w);
      mma_s8(c[nb], qf[2][0], qf[2][1], u1.x, u1.y);
      mma_s8(c[nb], qf[3][0], qf[3][1], u1.z, u1.w);
    } else {
      const uint4 u = *reinterpret_cast<const uint4*>(stage + nb * 512 + group * 64 + sub * 16);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int s = 0; s < 4; ++s) mma_s8(c[nb], qf[s][0], qf[s][1], (w[s] << 4) & 0xf0f0f0f0u, w[s] & 0xf0f0f0f0u);
    }
  }
  int acc[16];
#pragma unroll
  for (int nb = 0; nb < 8; ++nb) {
    acc[2 * nb] = K4 ? c[nb][0] >> 8 : c[nb][0];   // INT4: both operands were widened by 16
    acc[2 * nb + 1] = K4 ? c[nb][1] >> 8 : c[nb][1];
  }
  const bool ragged = key_begin + BN > prompt;       // only the last prompt tile has keys past the prompt
  unsigned live = row_on ? 0xffffu : 0u;
  if (ragged) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (key_begin + (i / 2) * 8 + sub * 2 + (i % 2) >= prompt) live &= ~(1u << i);
  }
  // scaled tile maximum: max over the 16-key groups of slope_c * max(acc) (slope_c > 0, so the order is free)
  float tmax = -CUDART_INF_F;
#pragma unroll
  for (int col = 0; col < 4; ++col) {
    int mi = INT_MIN;
#pragma unroll
    for (int i = 4 * col; i < 4 * col + 4; ++i)
      if ((live >> i) & 1u) mi = max(mi, acc[i]);
    if (mi != INT_MIN) tmax = fmaxf(tmax, qs * kt[col] * (float)mi);
  }
  tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
  tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
  const float tile = tmax;
  const float n = fmaxf(st.m, tile), alpha = exp2f(st.m - n);
  st.m = n;
  if (alpha != 1.f) {
#pragma unroll
    for (int cb = 0; cb < 16; ++cb) { st.out[cb][0] *= alpha; st.out[cb][1] *= alpha; }
    st.corr *= alpha;
  }
  constexpr float levels = V4 ? 15.f : 255.f;
  const bool any = tile > -CUDART_INF_F;
  const float slope1 = qs * fmaxf(fmaxf(kt[0], kt[1]), fmaxf(kt[2], kt[3]));
  float base = any ? tile : n;
  base += tile_base_margin(slope1, base);
  const float bq = any ? exp2f(base - n) / levels : 0.f, restore = V4 ? bq * (127.f / 7.f) : bq;
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float slope0 = qs * kt[i / 4];
    const int xbits = acc[i] + Magic;
    const float x = __int_as_float(xbits);
    const float bias = -slope0 * 12582912.f;
    const float arg = K4 ? fmaf(slope0, __fsub_rn(x, 12582912.f), -base) : fmaf(slope0, x, bias - base);
    const bool on = (live >> i) & 1u;
    w[i] = __float_as_uint(fmaf(on ? exp2f(arg) : 0.f, levels, on ? pmagic_dither(xbits) : 49152.f));
  }
  uint32_t pa[4];   // A fragments of P: a0/a2 of k-step 0, a0/a2 of k-step 1
#pragma unroll
  for (int j = 0; j < 4; ++j) pa[j] = pack_bytes(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  const int psum = (int)__dp4a(pa[0], 0x01010101u, __dp4a(pa[1], 0x01010101u, __dp4a(pa[2], 0x01010101u, __dp4a(pa[3], 0x01010101u, 0u))));
  st.denom = fmaf(st.denom, alpha, (float)psum * bq);
  if constexpr (!V4) st.corr = fmaf(12582912.f, restore, st.corr);
#pragma unroll
  for (int cb = 0; cb < 16; ++cb) {
    int d[4] = {0, 0, 0, 0};
    if constexpr (!V4) {
      const uint4 u = *reinterpret_cast<const uint4*>(vb + cb * 512 + group * 64 + sub * 16);
      mma_u8s8(d, pa[0], pa[1], u.x, u.y);
      mma_u8s8(d, pa[2], pa[3], u.z, u.w);
      st.out[cb][0] = fmaf(__int_as_float(d[0] + Magic), restore, st.out[cb][0]);
      st.out[cb][1] = fmaf(__int_as_float(d[1] + Magic), restore, st.out[cb][1]);
    } else {
      const uint2 u = *reinterpret_cast<const uint2*>(vb + cb * 256 + group * 32 + sub * 8);
      mma_u8s8(d, pa[0], pa[1], (u.x << 4) & 0xf0f0f0f0u, u.x & 0xf0f0f0f0u);
      mma_u8s8(d, pa[2], pa[3], (u.y << 4) & 0xf0f0f0f0u, u.y & 0xf0f0f0f0u);
      st.out[cb][0] = fmaf((float)(d[0] >> 4), restore, st.out[cb][0]);
      st.out[cb][1] = fmaf((float)(d[1] >> 4), restore, st.out[cb][1]);
    }
  }
}

// One 32-key chunk of an un-quantised BF16 head, whole warp (no counterpart in the reference).
__device__ __forceinline__ void bf16_chunk(const uint8_t* stage, const uint32_t (&qb)[8][2], float sm_log2, WarpState& st,
    int key_begin, int prompt, bool row_on) {
  const int lane = threadIdx.x % 32, group = lane / 4, sub = lane % 4;
  const uint8_t* vb = stage + 8192;
  float c[4][4];
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
    c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint4 x = *reinterpret_cast<const uint4*>(stage + (nb * 4 + u) * 512 + group * 64 + sub * 16);
      mma_bf16(c[nb], qb[2 * u][0], qb[2 * u][1], x.x, x.y);
      mma_bf16(c[nb], qb[2 * u + 1][0], qb[2 * u + 1][1], x.z, x.w);
    }
  }
  float s[8], tmax = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int key = key_begin + (i / 2) * 8 + sub * 2 + (i % 2);
    s[i] = (row_on && key < prompt) ? c[i / 2][i % 2] * sm_log2 : -CUDART_INF_F;
    tmax = fmaxf(tmax, s[i]);
  }
  tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
  tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
  const float n = fmaxf(st.m, tmax), alpha = exp2f(st.m - n);
  st.m = n;
  float p[8], part = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { p[i] = s[i] > -CUDART_INF_F ? exp2f(s[i] - n) : 0.f; part += p[i]; }
  st.denom = fmaf(st.denom, alpha, part);
  uint32_t pa[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(p[2 * j], p[2 * j + 1]);
    pa[j] = *reinterpret_cast<const uint32_t*>(&h);
  }
#pragma unroll
  for (int cb = 0; cb < 16; ++cb) {
    float o[4] = {st.out[cb][0] * alpha, st.out[cb][1] * alpha, 0.f, 0.f};
    const uint4 x = *reinterpret_cast<const uint4*>(vb + cb * 512 + group * 64 + sub * 16);
    mma_bf16(o, pa[0], pa[1], x.x, x.y);
    mma_bf16(o, pa[2], pa[3], x.z, x.w);
    st.out[cb][0] = o[0]; st.out[cb][1] = o[1];
  }
}

// Arguments of the merge (tail, statistics, output), passed by value to the kernel when the merge is fused.
struct MergeArgs {
  const int2* unit_slots; int32_t* unit_done;      // unit_done == nullptr: no fused merge
  float* fold_m; float* fold_l; float* fold_o;     // fold_m != nullptr: fold the unit's segments to one triple instead of merging
  // Sequence split with the exchange fused into the fold (peers != nullptr): the folded triple goes straight into the
  // exchange buffer of every GPU of the group by peer stores, followed by a flag.  See SplitExchange below.
  float* const* peers; int world, rank, units; int64_t rank_stride; int32_t* epoch;
  // present != nullptr: the CTA that delivered a unit's triple also waits for the other ranks' triples of the unit and
  // merges it (the whole sequence-split step is this one kernel); present[r * units + u] = rank r holds tiles of unit u.
  const int32_t* present;
  const float* vstat; const float* kstat;
  __nv_bfloat16* ktail; __nv_bfloat16* vtail; int64_t tsu, tst;
  const __nv_bfloat16* kcur; const __nv_bfloat16* vcur; int64_t csb, csh;
  const int64_t* step; __nv_bfloat16* out; int64_t osb, osh;
  int max_tail;
};

// ---- merge of one unit: split partials + BF16 tail -> output rows of its Q heads ------------------------------------
// Same arithmetic as decode_merge_kernel of the reference (common_device.cuh:373-469): tail scores q.(k - kmean) in fp32 on
// the un-rotated rows, base-2 maximum over partials and tail, de-normalisation of the cached part (acc * vscale +
// l * vmean), then the tail's exact P.V.  Shared by the stand-alone merge kernel (one CTA per unit) and by the decode
// kernel's CTA that finishes a unit (merge fused into the split pass).

// Tail scores of `nh` Q heads (rows qrows + i * qsh, i < nh) against the unit's tail, one pass over the tail's K rows:
// the `warps` calling warps split the rows, a lane holds 4 features of the row and of each head's q.  ts[i * ts_stride + t].
// (RowsLong also takes the first `staged` K rows from a copy in shared memory, ks, D elements per row: stage_tail_rows.)
// Rows picks how the row loop is compiled; the sums run in row order every way, so all give the same bits.  RowsShort: not
// unrolled, the first row comes back soonest (a step with a tail of a few rows; a long tail is then a chain of trips to
// memory).  RowsLong: unrolled so that several rows' loads are in flight.  RowsAny: left to the compiler (in between).
enum { RowsAny = 0, RowsShort = 1, RowsLong = 2 };
template <int V> struct IntConstant { static constexpr int value = V; };
template <int Rows = RowsAny>
__device__ __forceinline__ void unit_tail_scores(const __nv_bfloat16* qrows, int64_t qsh, int nh, const float* kmean_unit,
    const __nv_bfloat16* kt, int64_t tst, const __nv_bfloat16* kc, int prior, int tail, float sm_log2, float* ts, int ts_stride,
    int warp, int warps, int lane, const __nv_bfloat16* ks = nullptr, int staged = 0) {
  float qv[MaxGroup][4], kmean[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) kmean[i] = kmean_unit[lane * 4 + i];
#pragma unroll
  for (int r = 0; r < MaxGroup; ++r) {
    const __nv_bfloat16* qrow = qrows + (int64_t)min(r, nh - 1) * qsh + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) qv[r][i] = __bfloat162float(qrow[i]);
  }
  const auto row = [&](int t) {
    const __nv_bfloat16* kv = (t < prior ? kt + t * tst : kc) + lane * 4;
    float kd[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) kd[i] = __bfloat162float(kv[i]) - kmean[i];
#pragma unroll
    for (int r = 0; r < MaxGroup; ++r) {
      if (r < nh) {
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) part = fmaf(qv[r][i], kd[i], part);
#pragma unroll
        for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) ts[r * ts_stride + t] = part * sm_log2;
      }
    }
  };
  if constexpr (Rows == RowsShort) {
#pragma unroll 1
    for (int t = warp; t < tail; t += warps) row(t);
  } else if constexpr (Rows == RowsLong) {
    // Four heads' lane sums reduced together: after the exchange over 16 lanes a lane carries two heads, after the one
    // over 8 lanes one, so a row costs six shuffles per four heads instead of twenty, in one chain of five, with no
    // branch between rows.  Every sum adds the same two operands as the butterfly of the plain loop does in lane 0
    // (addition commutes, so all lanes of a butterfly hold the same bits): the scores are bit-equal.
    const bool up16 = lane & 16, up8 = lane & 8;
    const int mine = ((lane >> 3) & 1) + 2 * ((lane >> 4) & 1);
    const auto quad = [&](int t, const float (&kd)[4], auto first) {
      constexpr int r0 = decltype(first)::value;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) v[j] = fmaf(qv[r0 + j][i], kd[i], v[j]);
      }
      const float w0 = (up16 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, up16 ? v[0] : v[2], 16);
      const float w1 = (up16 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, up16 ? v[1] : v[3], 16);
      float x = (up8 ? w1 : w0) + __shfl_xor_sync(0xffffffffu, up8 ? w0 : w1, 8);
#pragma unroll
      for (int o = 4; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
      if ((lane & 7) == 0 && r0 + mine < nh) ts[(r0 + mine) * ts_stride + t] = x * sm_log2;
    };
#pragma unroll 4
    for (int t = warp; t < tail; t += warps) {   // the first `staged` rows from their copy in shared memory (ks)
      const __nv_bfloat16* kv = (t < staged ? ks + t * D : t < prior ? kt + t * tst : kc) + lane * 4;
      float kd[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) kd[i] = __bfloat162float(kv[i]) - kmean[i];
      quad(t, kd, IntConstant<0>{});
      if (nh > 4) quad(t, kd, IntConstant<4>{});
    }
  } else {
    for (int t = warp; t < tail; t += warps) row(t);
  }
}

// Copy of the first min(tail, limit) rows of a unit's tail (row t < prior from the tail buffer, row `prior` = this step's
// row from the caller's tensor) into shared memory, D elements per row, by asynchronous 8-byte copies of all `threads`
// calling threads (the alignment the row loops assume anyway); returns the number of rows.  The copies are complete for
// the CTA after stage_tail_wait() and a barrier.
__device__ __forceinline__ int stage_tail_rows(__nv_bfloat16* dst, const __nv_bfloat16* rows, int64_t tst, const __nv_bfloat16* current,
                                               int prior, int tail, int limit, int tid, int threads) {
  const int n = min(tail, limit);
  for (int i = tid; i < n * (D / 4); i += threads) {
    const int t = i / (D / 4), piece = i % (D / 4);
    const __nv_bfloat16* src = (t < prior ? rows + (int64_t)t * tst : current) + piece * 4;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst + t * D + piece * 4)), "l"(src) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  return n;
}
__device__ __forceinline__ void stage_tail_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// One warp merges one Q head: nsplit partials at pm[first + s * ml_stride], pl likewise, po[first * 128 + s * o_stride + ch]
// (a lane holds 4 of the 128 channels), the tail scores of the head in ts_row[0 .. tail) (turned into weights in place),
// the tail's V rows, and writes the head's output row.  Partials are read past L1 (they may come from other CTAs of the
// same launch or from other GPUs), four splits' loads in flight at a time; the sums run in split order.
// Rows: as for unit_tail_scores.  RowsLong also takes the first `staged` V rows of the tail from a copy in shared memory
// (vs, D elements per row; stage_tail_rows), the rest from where they lie.
template <int Rows = RowsAny>
__device__ __forceinline__ void merge_head_by_warp(const float* pm, const float* pl, const float* po, int64_t first,
    int64_t ml_stride, int64_t o_stride, int nsplit, float* ts_row, int tail, int prior, const __nv_bfloat16* vt, int64_t tst,
    const __nv_bfloat16* vc, const float* vstat_unit, __nv_bfloat16* out_row, int lane, const __nv_bfloat16* vs = nullptr,
    int staged = 0) {
  // The first four splits' (m, l, o) are requested at once, before the maximum is known: their addresses depend on
  // nothing that is computed here, so the merge pays one trip to the second-level cache instead of two (a unit seldom
  // has more than four splits).
  float pmv[4], plv[4];
  float4 p[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const bool on = u < nsplit;
    pmv[u] = on ? __ldcg(pm + first + u * ml_stride) : -FLT_MAX;
    plv[u] = on ? __ldcg(pl + first + u * ml_stride) : 0.f;
    p[u] = on ? __ldcg(reinterpret_cast<const float4*>(po + first * D + u * o_stride + lane * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m = -FLT_MAX;
  for (int s = 4 + lane; s < nsplit; s += 32) m = fmaxf(m, __ldcg(pm + first + s * ml_stride));
  for (int t = lane; t < tail; t += 32) m = fmaxf(m, ts_row[t]);
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  m = fmaxf(fmaxf(m, fmaxf(pmv[0], pmv[1])), fmaxf(pmv[2], pmv[3]));
  for (int t = lane; t < tail; t += 32) ts_row[t] = exp2f(ts_row[t] - m);
  __syncwarp();
  float total = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s0 = 0; s0 < nsplit; s0 += 4) {
    if (s0 > 0) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool on = s0 + u < nsplit;
        pmv[u] = on ? __ldcg(pm + first + (s0 + u) * ml_stride) : -FLT_MAX;
        plv[u] = on ? __ldcg(pl + first + (s0 + u) * ml_stride) : 0.f;
        p[u] = on ? __ldcg(reinterpret_cast<const float4*>(po + first * D + (s0 + u) * o_stride + lane * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (s0 + u < nsplit) {
        const float w = exp2f(pmv[u] - m);
        total = fmaf(plv[u], w, total);
        acc[0] = fmaf(p[u].x, w, acc[0]); acc[1] = fmaf(p[u].y, w, acc[1]); acc[2] = fmaf(p[u].z, w, acc[2]); acc[3] = fmaf(p[u].w, w, acc[3]);
      }
    }
  }
  const float4 mean = *reinterpret_cast<const float4*>(vstat_unit + lane * 4);
  const float4 scale = *reinterpret_cast<const float4*>(vstat_unit + D + lane * 4);
  acc[0] = acc[0] * scale.x + total * mean.x; acc[1] = acc[1] * scale.y + total * mean.y;
  acc[2] = acc[2] * scale.z + total * mean.z; acc[3] = acc[3] * scale.w + total * mean.w;
  const auto add = [&](int t, const __nv_bfloat16* v) {
    const float e = ts_row[t];
    const uint2 raw = *reinterpret_cast<const uint2*>(v + lane * 4);
    const float2 v01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 v23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    total += e;
    acc[0] = fmaf(e, v01.x, acc[0]); acc[1] = fmaf(e, v01.y, acc[1]); acc[2] = fmaf(e, v23.x, acc[2]); acc[3] = fmaf(e, v23.y, acc[3]);
  };
  const auto row = [&](int t) { add(t, t < prior ? vt + (int64_t)t * tst : vc); };
  if constexpr (Rows == RowsShort) {
#pragma unroll 1
    for (int t = 0; t < tail; ++t) row(t);
  } else if constexpr (Rows == RowsLong) {
#pragma unroll 8
    for (int t = 0; t < staged; ++t) add(t, vs + t * D);
#pragma unroll 16
    for (int t = staged; t < tail; ++t) row(t);
  } else {
    for (int t = 0; t < tail; ++t) row(t);
  }
  const __nv_bfloat162 o01 = __floats2bfloat162_rn(acc[0] / total, acc[1] / total);
  const __nv_bfloat162 o23 = __floats2bfloat162_rn(acc[2] / total, acc[3] / total);
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t*>(&o01);
  packed.y = *reinterpret_cast<const uint32_t*>(&o23);
  *reinterpret_cast<uint2*>(out_row + lane * 4) = packed;
}

// Merge of one unit by the consumer warps of the decode kernel's CTA that finished the unit's last segment, with the
// CTA's fold buffer as scratch for the tail scores: up to ConsumerWarps Q heads per round, one warp per head.
// All ConsumerWarps*32 threads call it.  Partials: split s of head r at pm[(first*8 + r) + s*ml_stride] (see
// decode_merge_kernel).
// part = 0: everything; 1: only what does not need the partials (the tail append and, when all Q heads fit one round, their
// tail scores), returning whether the scores are in `scratch`; 2: the rest, given that part 1 returned true.  Splitting it
// lets the CTA do part 1 while the other GPUs' triples are still on their way.
__device__ __forceinline__ bool merge_unit_by_consumers(const MergeArgs& a, const float* pm, const float* pl, const float* po,
    int64_t first_slot, int64_t ml_stride, int64_t o_stride, int nsplit, const __nv_bfloat16* q, int64_t qsb, int64_t qsh,
    int unit, int heads_kv, int g, float sm_log2, float* scratch, int part = 0) {
  const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
  const int b = unit / heads_kv, kh = unit % heads_kv;
  const int prior = min((int)*a.step, a.max_tail - 1), tail = prior + 1;
  const __nv_bfloat16* kc = a.kcur + b * a.csb + kh * a.csh;
  const __nv_bfloat16* vc = a.vcur + b * a.csb + kh * a.csh;
  __nv_bfloat16* kt = a.ktail + unit * a.tsu;
  __nv_bfloat16* vt = a.vtail + unit * a.tsu;
  if (part != 2 && tid < D) {   // append the current token to the tail (read back only by later steps)
    kt[prior * a.tst + tid] = kc[tid];
    vt[prior * a.tst + tid] = vc[tid];
  }
  const int per_round = min(min(g, ConsumerWarps), (ConsumerWarps * CombFloats) / tail);   // >= 6 for tails up to 1024 rows
  if (part == 1 && per_round < g) return false;
  for (int h0 = 0; h0 < g; h0 += per_round) {
    const int nh = min(per_round, g - h0);
    const __nv_bfloat16* qrows = q + b * qsb + (int64_t)(kh * g + h0) * qsh;
    if (part != 2)
      unit_tail_scores(qrows, qsh, nh, a.kstat + (int64_t)unit * StatFloats, kt, a.tst, kc, prior, tail, sm_log2, scratch, tail,
                       warp, ConsumerWarps, lane);
    if (part == 1) return true;    // (the caller's next barrier orders the scores before part 2 reads them)
    consumer_sync();
    if (warp < nh)
      merge_head_by_warp(pm, pl, po, first_slot * MaxGroup + h0 + warp, ml_stride, o_stride, nsplit, scratch + warp * tail, tail,
                         prior, vt, a.tst, vc, a.vstat + (int64_t)unit * StatFloats,
                         a.out + b * a.osb + (int64_t)(kh * g + h0 + warp) * a.osh, lane);
    consumer_sync();   // scratch is reused by the next round (and by the next segment's fold)
  }
  return true;
}

// ---- exchange of folded triples between the GPUs of a sequence-split group, over peer memory ----------------------
// Every GPU owns one exchange buffer of the same layout, mapped into all the others (symmetric memory):
//   float data[2][world][rank_stride]   parity of the step's epoch, source rank, then that rank's [m | l | o] block
//                                       (m, l: [units][8]; o: [units][8][128]; rank_stride = units * 8 * 130)
//   int   flag[world][units]            the last epoch for which source rank's triple of the unit is complete
// A unit's epoch counts the decode steps: the folding CTA keeps it in `epoch[unit]` (local memory), the merging CTA in
// its own counter; both advance by one per step on every GPU.  The producer writes the triple into block
// [epoch & 1][its rank] of EVERY GPU's buffer (plain stores through NVLink), fences, and then stores the epoch into
// flag[its rank][unit] there.  The consumer (the merge kernel's CTA of that unit) waits, with a time limit, until the
// flags of all source ranks have reached its epoch and reads the parity's blocks from its own buffer.  Two parities
// are enough: a GPU cannot fold step e+1 before its own merge of step e is done, which needed every other GPU's fold of
// step e, which came after that GPU's merge of step e-1.
__device__ __forceinline__ int32_t load_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int64_t exchange_flag_offset(int world, int64_t rank_stride) { return 2 * (int64_t)world * rank_stride; }

// Fold of one unit by the consumer warps of the CTA that finished the unit's last segment: one (m, l, o) per
// Q head from the unit's segment partials, written at [unit][MaxGroup] of the fold buffers.  Used when a unit's
// tile range is split across GPUs: the folded triples are what the ranks exchange.  Same arithmetic and order as
// decode_fold_kernel; no V de-normalisation, no tail.
__device__ __forceinline__ void fold_unit_by_consumers(const MergeArgs& a, const float* pm, const float* pl, const float* po,
    int unit, int g) {
  const int2 sl = a.unit_slots[unit];
  // One item = (Q head r, 4 channels).  The partials come from other CTAs (read past L1); a segment's three loads
  // depend on nothing but the segment number, so they are issued four segments at a time and the latency of the
  // second-level cache is paid once per batch instead of once per segment.  The sums run in segment order.
  for (int e = threadIdx.x; e < g * (D / 4); e += ConsumerWarps * 32) {
    const int r = e / (D / 4), ch = (e % (D / 4)) * 4;
    const float* m0 = pm + (int64_t)sl.x * MaxGroup + r;
    const float* l0 = pl + (int64_t)sl.x * MaxGroup + r;
    const float* o0 = po + ((int64_t)sl.x * MaxGroup + r) * D + ch;
    float big = -FLT_MAX;
    for (int s0 = 0; s0 < sl.y; s0 += 4) {
      float m[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) m[u] = s0 + u < sl.y ? __ldcg(m0 + (int64_t)(s0 + u) * MaxGroup) : -FLT_MAX;
#pragma unroll
      for (int u = 0; u < 4; ++u) big = fmaxf(big, m[u]);
    }
    float o[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
    for (int s0 = 0; s0 < sl.y; s0 += 4) {
      float m[4], pl4[4];
      float4 p[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool on = s0 + u < sl.y;
        m[u] = on ? __ldcg(m0 + (int64_t)(s0 + u) * MaxGroup) : -FLT_MAX;
        pl4[u] = on ? __ldcg(l0 + (int64_t)(s0 + u) * MaxGroup) : 0.f;
        p[u] = on ? __ldcg(reinterpret_cast<const float4*>(o0 + (int64_t)(s0 + u) * MaxGroup * D)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u < sl.y) {
          const float w = exp2f(m[u] - big);
          o[0] = fmaf(p[u].x, w, o[0]); o[1] = fmaf(p[u].y, w, o[1]); o[2] = fmaf(p[u].z, w, o[2]); o[3] = fmaf(p[u].w, w, o[3]);
          l = fmaf(pl4[u], w, l);
        }
      }
    }
    const int64_t dst = (int64_t)unit * MaxGroup + r;
    if (a.peers == nullptr) {
      *reinterpret_cast<float4*>(a.fold_o + dst * D + ch) = make_float4(o[0], o[1], o[2], o[3]);
      if (ch == 0) { a.fold_m[dst] = big; a.fold_l[dst] = l; }
    } else {
      // straight into every GPU's exchange buffer: block [parity of this unit's next epoch][this rank]
      const int parity = (a.epoch[unit] + 1) & 1;
      const int64_t ug = (int64_t)a.units * MaxGroup;
      const int64_t block = ((int64_t)parity * a.world + a.rank) * a.rank_stride;
      for (int p = 0; p < a.world; ++p) {
        float* base = a.peers[p] + block;
        *reinterpret_cast<float4*>(base + 2 * ug + dst * D + ch) = make_float4(o[0], o[1], o[2], o[3]);
        if (ch == 0) { base[dst] = big; base[ug + dst] = l; }
      }
    }
  }
  if (a.peers != nullptr) {
    // All threads' peer stores, then the barrier, then ONE system-wide fence by the thread that raises the flags: the
    // fence is cumulative over what the barrier made visible to that thread (the pattern of a grid-wide barrier), so a
    // GPU that sees the flag sees the triple; one NVLink round trip instead of one per thread and per flag.
    consumer_sync();
    if (threadIdx.x == 0) {
      const int e = a.epoch[unit] + 1;
      a.epoch[unit] = e;
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) {
        volatile int32_t* flags = reinterpret_cast<volatile int32_t*>(a.peers[p] + exchange_flag_offset(a.world, a.rank_stride));
        flags[(int64_t)a.rank * a.units + unit] = e;
      }
    }
  }
}

// grid = persistent CTAs (one per SM), 224 threads.  cta_seg[c]..cta_seg[c+1] indexes the CTA's
// segments; segs[j] = {unit, first kept tile, tile count, partial slot}; unit = sequence*heads_kv + kv head.
__global__ void __launch_bounds__(DecodeThreads, 1) decode_kernel(const __nv_bfloat16* q, int64_t qsb, int64_t qsh,
    const uint8_t* pool, const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_flags, const int2* tmeta,
    const int4* segs, const int32_t* cta_seg, float* pm, float* pl, float* po, int heads_q, int heads_kv, int prompt_keys,
    float sm_log2, int stream_only, int slot_limit, MergeArgs margs, int* err) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[DecodeStages], empty[DecodeStages];
  __shared__ uint32_t stage_info[DecodeStages];

  __shared__ int abort_flag, merge_flag;
  const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32, group = lane / 4, sub = lane % 4;
  const int seg0 = cta_seg[blockIdx.x], nseg = cta_seg[blockIdx.x + 1] - seg0;
  const int g = heads_q / heads_kv;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < DecodeStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_fence_init();
    abort_flag = 0;
  }

  __syncthreads();
  // Up to here the CTA touched only its own shared memory and the plan tables; the cache, Q and the
  // partial buffers (which the previous step's merge may still be reading) come after the wait.
  grid_dependency_wait();
  grid_launch_dependents();
  volatile int* abortp = &abort_flag;

  if (warp == ConsumerWarps) {
    // ---- producer warp: keeps the ring full ----------------------------------------------------------
    // The tile table is read 32 entries at a time (one coalesced load per lane, the next batch in
    // flight while the current one is issued), so no global-memory latency sits between two copies;
    // lane 0 waits for a free stage and issues the bulk copy.
    int t = 0;
    for (int j = 0; j < nseg && !*abortp; ++j) {
      const int4 sg = segs[seg0 + j];
      const int2* meta = tmeta + unit_tab[sg.x] + sg.y;
      const uint8_t* base = pool + unit_base[sg.x];
      int2 batch = lane < sg.z ? meta[lane] : make_int2(0, 0);
      for (int i0 = 0; i0 < sg.z && !*abortp; i0 += 32) {
        const int2 next = i0 + 32 + lane < sg.z ? meta[i0 + 32 + lane] : make_int2(0, 0);
        const int nb = min(32, sg.z - i0);
        for (int k = 0; k < nb; ++k, ++t) {
          const int off16 = __shfl_sync(0xffffffffu, batch.x, k), info = __shfl_sync(0xffffffffu, batch.y, k);
          if (lane == 0) {
            const int s = t % DecodeStages;
            if (mbar_wait_abortable(&empty[s], ((t / DecodeStages) & 1) ^ 1, abortp)) {
              const uint32_t bytes = chunk_bytes((uint32_t)info);
              stage_info[s] = (uint32_t)info;
              mbar_expect_tx(&full[s], bytes);
              bulk_g2s(smem + SmRing + s * StageBytes, base + (int64_t)off16 * 16, bytes, &full[s]);
            }
          }
        }
        batch = next;
      }
    }
  } else {
    // ---- consumers: warp w owns tiles t = w, w + ConsumerWarps, ... of the CTA's list -----------------
    uint8_t* q8buf = smem + SmComb + warp * CombFloats * 4;
    uint8_t* q4buf = q8buf + 1024;
    float* comb = reinterpret_cast<float*>(smem + SmComb);
    int t0 = 0;
    for (int j = 0; j < nseg; ++j) {
      const int4 sg = segs[seg0 + j];
      const int unit = sg.x, count = sg.z, slot = sg.w;
      const int b = unit / heads_kv, kh = unit % heads_kv;
      const bool bf16 = unit_flags[unit] & 1;
      const __nv_bfloat16* qrow = q + b * qsb + (int64_t)(kh * g) * qsh;
      uint32_t qf[4][2], qf4[4][2], qb[8][2];
      float qs8 = FLT_MIN, qs4 = FLT_MIN;
      if (!bf16) {
        // Q of the group: rotate + quantise, one row at a time with the reference's lane mapping
        // (common_device.cuh:291-315), then gather this lane's fragments through shared memory.
        __syncwarp();
        for (int r = 0; r < MaxGroup; ++r) {
          uint32_t word = 0, word4 = 0;
          if (r < g) {
            float xv[4], mxq = 0.f;
            const __nv_bfloat16* src = qrow + r * qsh + lane * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = __bfloat162float(src[i]);
            rotate128_x4(xv, lane);
#pragma unroll
            for (int i = 0; i < 4; ++i) mxq = fmaxf(mxq, fabsf(xv[i]));
#pragma unroll
            for (int o = 16; o; o >>= 1) mxq = fmaxf(mxq, __shfl_xor_sync(0xffffffffu, mxq, o));
            const float inv = mxq > 0.f ? 127.f / mxq : 0.f, inv4 = mxq > 0.f ? 7.f / mxq : 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              word |= (uint32_t)(__float2int_rn(xv[i] * inv) & 0xff) << (8 * i);
              word4 |= (uint32_t)((__float2int_rn(xv[i] * inv4) & 0xf) << 4) << (8 * i);   // code * 16 as int8
            }
            if (group == r) {
              qs8 = mxq > 0.f ? mxq / 127.f * sm_log2 : FLT_MIN;
              qs4 = mxq > 0.f ? mxq / 7.f * sm_log2 : FLT_MIN;
            }
          }
          reinterpret_cast<uint32_t*>(q8buf + r * D)[lane] = word;
          reinterpret_cast<uint32_t*>(q4buf + r * D)[lane] = word4;
        }
        __syncwarp();
#pragma unroll
        for (int s = 0; s < 4; ++s) {   // k-step s, positions 4sub+j -> feature 32sub+8s+j, 16+4sub+j -> +4
          qf[s][0] = *reinterpret_cast<const uint32_t*>(q8buf + group * D + sub * 32 + s * 8);
          qf[s][1] = *reinterpret_cast<const uint32_t*>(q8buf + group * D + sub * 32 + s * 8 + 4);
          qf4[s][0] = *reinterpret_cast<const uint32_t*>(q4buf + group * D + sub * 32 + s * 8);
          qf4[s][1] = *reinterpret_cast<const uint32_t*>(q4buf + group * D + sub * 32 + s * 8 + 4);
        }
      } else {
#pragma unroll
        for (int fs = 0; fs < 8; ++fs) {   // k-step fs: features 32sub + 4fs + {0,1} and + {2,3}
          qb[fs][0] = group < g ? *reinterpret_cast<const uint32_t*>(qrow + group * qsh + sub * 32 + fs * 4) : 0u;
          qb[fs][1] = group < g ? *reinterpret_cast<const uint32_t*>(qrow + group * qsh + sub * 32 + fs * 4 + 2) : 0u;
        }
      }
      WarpState st;
      st.m = -FLT_MAX; st.denom = 0.f; st.corr = 0.f;
#pragma unroll
      for (int cb = 0; cb < 16; ++cb) st.out[cb][0] = st.out[cb][1] = 0.f;

      int first_t = t0 + ((warp - t0 % ConsumerWarps) + ConsumerWarps) % ConsumerWarps;
      for (int t = first_t; t < t0 + count; t += ConsumerWarps) {
        const int s = t % DecodeStages;
        if (!mbar_wait_abortable(&full[s], (t / DecodeStages) & 1, abortp)) break;
        const uint8_t* stage = smem + SmRing + s * StageBytes;
        const uint32_t info = stage_info[s];
        const int tile = info & InfoTileMask;
        const unsigned rowmask = (info >> InfoRowShift) & 0xffu;
        const bool row_on = group < g && ((rowmask >> group) & 1u);
        const int prompt = (info & InfoFull) ? 0x7fffffff : prompt_keys;
        if (stream_only) {
          // diagnostic: consume the ring without arithmetic (measures the copy pipeline alone)
        } else if (info & InfoBf16) {
          bf16_chunk(stage, qb, sm_log2, st, tile * Bf16ChunkKeys, prompt, row_on);
        } else if (info & InfoK4) {
          if (info & InfoV4) quantised_tile<true, true>(stage, qf4, qs4, st, tile * BN, prompt, row_on);
          else quantised_tile<true, false>(stage, qf4, qs4, st, tile * BN, prompt, row_on);
        } else {
          if (info & InfoV4) quantised_tile<false, true>(stage, qf, qs8, st, tile * BN, prompt, row_on);
          else quantised_tile<false, false>(stage, qf, qs8, st, tile * BN, prompt, row_on);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);   // the stage may be refilled
      }
      t0 += count;

      // ---- fold the consumer warps' states of this segment into one partial (m, l, o) per Q head ---
      float den = st.denom;
      den += __shfl_xor_sync(0xffffffffu, den, 1);
      den += __shfl_xor_sync(0xffffffffu, den, 2);
      float* mine = comb + warp * CombFloats;
#pragma unroll
      for (int cb = 0; cb < 16; ++cb)
        *reinterpret_cast<float2*>(mine + group * D + cb * 8 + sub * 2) = make_float2(st.out[cb][0] - st.corr, st.out[cb][1] - st.corr);
      if (sub == 0) { mine[MaxGroup * D + group] = st.m; mine[MaxGroup * D + MaxGroup + group] = den; }
      consumer_sync();
      if (slot < 0 || slot >= slot_limit) {
        // a plan whose slot column does not fit the partial buffers: record it and store nothing
        if (tid == 0) atomicCAS(err, ErrNone, ErrBadSlot);
      } else {
        for (int e = tid; e < g * D; e += ConsumerWarps * 32) {   // one (Q head, channel) per consumer thread
          const int r = e / D, ch = e % D;
          float mw[ConsumerWarps], big = -FLT_MAX;
#pragma unroll
          for (int w = 0; w < ConsumerWarps; ++w) { mw[w] = comb[w * CombFloats + MaxGroup * D + r]; big = fmaxf(big, mw[w]); }
          float o = 0.f, l = 0.f;
#pragma unroll
          for (int w = 0; w < ConsumerWarps; ++w) {
            const float sc = exp2f(mw[w] - big);
            o = fmaf(comb[w * CombFloats + r * D + ch], sc, o);
            l = fmaf(comb[w * CombFloats + MaxGroup * D + MaxGroup + r], sc, l);
          }
          const int64_t idx = (int64_t)slot * MaxGroup + r;
          po[idx * D + ch] = o;
          if (ch == 0) { pm[idx] = big; pl[idx] = l; }
        }
      }
      consumer_sync();   // the fold buffer is free for the next segment; every consumer thread's stores of the partial are done
      if (margs.unit_done != nullptr) {
        // Fused merge: whoever finishes a unit's last segment merges the unit (its partials, the BF16 tail
        // and the output) right here, while the producer warp keeps prefetching the next segment.
        if (tid == 0) {
          // One fence for the CTA: the barrier ordered the other threads' stores before it, and a fence is cumulative, so
          // the partial is visible device-wide before the count moves (192 fences per segment cost microseconds).
          __threadfence();
          const int done = atomicAdd(&margs.unit_done[unit], 1);
          const int last = done == margs.unit_slots[unit].y - 1;
          if (last) margs.unit_done[unit] = 0;   // ready for the next launch
          merge_flag = last;
        }
        consumer_sync();
        if (merge_flag) {
          __threadfence();
          const int2 sl = margs.unit_slots[unit];
          if (sl.x < 0 || sl.y < 0 || sl.x + sl.y > slot_limit) {
            if (tid == 0) atomicCAS(err, ErrNone, ErrBadSlot);
          } else if (margs.fold_m != nullptr || margs.peers != nullptr) {
            fold_unit_by_consumers(margs, pm, pl, po, unit, g);
            if (margs.peers != nullptr && margs.present != nullptr) {
              // This GPU's triple of the unit is on its way to every GPU of the group.  Wait (at most one second) for
              // theirs, then merge the unit here: the exchange and the merge cost no further launch.  The producer warp
              // keeps prefetching this CTA's next tiles meanwhile.
              if (tid == 0) merge_flag = 0;
              consumer_sync();                      // (also makes epoch[unit], just advanced by thread 0, visible)
              const int e = margs.epoch[unit];
              float* local = margs.peers[margs.rank];
              // what the merge needs besides the triples (tail append, tail scores) is done while they travel
              const bool scored = merge_unit_by_consumers(margs, nullptr, nullptr, nullptr, 0, 0, 0, 0, q, qsb, qsh, unit, heads_kv, g,
                                                          sm_log2, comb, 1);
              if (tid < margs.world && tid != margs.rank && margs.present[(int64_t)tid * margs.units + unit]) {
                const int32_t* flag = reinterpret_cast<const int32_t*>(local + exchange_flag_offset(margs.world, margs.rank_stride)) +
                                      (int64_t)tid * margs.units + unit;
                const uint64_t t_wait = globaltimer_ns();
                while (load_acquire_sys(flag) < e) {
                  if (globaltimer_ns() - t_wait > 1000000000ull) { merge_flag = 1; break; }
                }
              }
              consumer_sync();
              if (merge_flag) {
                if (tid == 0) atomicCAS(err, ErrNone, ErrBarrierTimeout);
              } else {
                const float* block = local + (int64_t)(e & 1) * margs.world * margs.rank_stride;
                const int64_t ug = (int64_t)margs.units * MaxGroup;
                merge_unit_by_consumers(margs, block, block + ug, block + 2 * ug, unit, margs.rank_stride, margs.rank_stride,
                                        margs.world, q, qsb, qsh, unit, heads_kv, g, sm_log2, comb, scored ? 2 : 0);
              }
            }
          } else {
            merge_unit_by_consumers(margs, pm, pl, po, sl.x, MaxGroup, (int64_t)MaxGroup * D, sl.y, q, qsb, qsh, unit, heads_kv, g,
                                    sm_log2, comb);
          }
        }
      }
    }
  }
  if (*abortp) {
    // a wait ran out: give copies that may still be in flight a bounded time to land before the CTA
    // (and its shared memory) goes away
    const uint64_t t_abort = globaltimer_ns();
    while (globaltimer_ns() - t_abort < 2000000ull) {}
  }
  __syncthreads();
  if (tid == 0 && abort_flag) atomicExch(err, ErrBarrierTimeout);
}

}  // namespace tri
