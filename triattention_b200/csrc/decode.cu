// Split-KV decode over the mixed-width KV cache, sm_100a: host launchers, the merge kernel and the
// cache-store (gather + re-layout) kernels.  The streaming kernel itself is in decode_kernel.cuh.
//
// Replaces (paths inside the reference project)
//   triattention/kernels/cuda/common_device.cuh:178-371  decode_tile, decode_kernel
//   triattention/kernels/cuda/common_device.cuh:373-469  decode_merge_kernel
//   triattention/kernels/cuda/common_host.cuh:47-94      decode, decode_occupancy
//   triattention/kernels/decode.py:46-61                 the index_select gathers of DecodeCache.store
// with a batch dimension, a cost-balanced static partition of the tile sequence over persistent CTAs
// instead of a fixed tiles-per-split, and an un-quantised BF16 head kind that the reference lacks.
#include "decode_kernel.cuh"
#include "abi_internal.h"

namespace tri {

// ---- merge: split partials + BF16 tail -> output, one CTA per (sequence, KV head) unit -------------------
// Replaces decode_merge_kernel of the reference (common_device.cuh:373-469: one CTA per Q head), same arithmetic:
// tail scores q.(k - kmean) in fp32 on the un-rotated rows, base-2 running maximum over partials and tail,
// de-normalisation of the cached part (acc * vscale + l * vmean), then the tail's exact P.V.
// Organisation: grid = units, 8 warps.  The unit's tail K rows are read ONCE for all g Q heads of the group
// (warps split the rows, a lane holds 4 features of the row and of each head's q); after that warp r owns Q head
// r: it walks the unit's partials (a lane holds 4 of the 128 channels, so one partial is one 512-byte row per
// warp) and then the tail's V rows, and writes its head's output row.
// Partials are addressed as pm[first * 8 + s * ml_stride + r], po[(first * 8 + r) * 128 + s * o_stride + ch] for
// split s of the unit: ml_stride = 8, o_stride = 1024 for the dense [slot][8] buffers of the split pass; other
// strides let the merge read triples gathered from several GPUs in place ([rank][unit][8]).
constexpr int MergeThreads = 256, MergeWarps = MergeThreads / 32;
// Consumer side of the peer-memory exchange of a sequence-split group (decode_kernel.cuh): world > 0 makes the unit's CTA
// wait until every source rank that holds tiles of the unit (present[rank][unit]) has delivered the triple of this
// unit's next epoch into the local exchange buffer, and read the partials from that epoch's parity block.
struct SplitExchange {
  const float* local; const int32_t* present; int32_t* seen; int world, units; int64_t rank_stride;
};
// Output gather by peer stores (unit sharding across GPUs): world > 0 makes every Q-head row go, instead of into `out`,
// into the full output tensor of EVERY GPU of the group, at the row the (sequence, head) has there.  peers[r] = rank r's
// gather buffer as mapped here: bf16 data [2][rows_total][128] (parity of the step, then the full [B, Hq] rows) followed
// by int32 flags [world] (64-byte aligned).  unit_row[u] = row of the unit's first Q head in the full tensor.
// sync[0] counts finished CTAs of the launch, sync[1] the steps done (the epoch).  The CTA that finishes last raises
// flag[rank] = epoch on every GPU; gather_wait_kernel is the consumer.
struct OutputGather {
  void* const* peers; const int64_t* unit_row; int32_t* sync; int world, rank; int64_t rows_total;
};
__device__ __forceinline__ int64_t gather_flag_offset_bytes(int64_t rows_total) { return (2 * rows_total * D * 2 + 63) / 64 * 64; }
// Two instantiations, the same arithmetic in the same order: LongTail = false for steps whose BF16 tail has a few rows
// (row loops not unrolled: 5 us per step less at one row, 100 us more at 256 rows), LongTail = true for the rest (row
// loops unrolled; 3 us ahead from 16 rows on; the tail's first StagedTailRows K rows, and after the scores its V rows,
// copied into dynamic shared memory by the whole CTA in one go, so that a row costs no trip to memory of its own and
// the g warps that walk the V rows in order do not each fetch them).  The host picks one per launch from the caller's hint (tri_decode_tail_hint); a separate kernel and not
// a branch, because any more code inside this kernel made its one-row case slower.
constexpr int StagedTailRows = 256;
constexpr int StagedTailBytes = StagedTailRows * D * 2;
template <bool LongTail>
__global__ void __launch_bounds__(MergeThreads) decode_merge_kernel(const float* pm, const float* pl, const float* po,
    int64_t ml_stride, int64_t o_stride, SplitExchange xchg, OutputGather gather, const int2* unit_slots, int slot_limit,
    const float* vstat, const float* kstat,
    const __nv_bfloat16* q, int64_t qsb, int64_t qsh, __nv_bfloat16* ktail, __nv_bfloat16* vtail, int64_t tsu, int64_t tst,
    const __nv_bfloat16* kcur, const __nv_bfloat16* vcur, int64_t csb, int64_t csh, const int64_t* step, __nv_bfloat16* out,
    int64_t osb, int64_t osh, int heads_q, int heads_kv, int max_tail, float sm_log2, int* err) {
  __shared__ float ts[MaxGroup][1024];   // tail scores, then tail weights, per Q head of the group
  const int unit = blockIdx.x, b = unit / heads_kv, kh = unit % heads_kv, g = heads_q / heads_kv;
  const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
  grid_launch_dependents();   // the next step's split pass may set up its barriers behind this kernel
  const int2 sl = unit_slots[unit];
  if (sl.x < 0 || sl.y < 0 || sl.x + sl.y > slot_limit) {   // the unit's slots do not fit the partial buffers
    if (tid == 0) atomicCAS(err, ErrNone, ErrBadSlot);
    return;
  }
  // What does not depend on the split pass comes before the wait for it: the tail append and the tail scores read only
  // this step's q / k / v, the statistics and the tail rows of earlier steps, all complete before the split pass began
  // (it waited for its own predecessor before it let this kernel start), so a CTA that becomes resident while other SMs
  // still stream has only the partials left to read afterwards.
  const int prior = min((int)*step, max_tail - 1), tail = prior + 1;
  const __nv_bfloat16* kc = kcur + b * csb + kh * csh;
  const __nv_bfloat16* vc = vcur + b * csb + kh * csh;
  __nv_bfloat16* kt = ktail + unit * tsu;
  __nv_bfloat16* vt = vtail + unit * tsu;
  if (tid < D) {   // append the current token to the tail (read back only by later steps)
    kt[prior * tst + tid] = kc[tid];
    vt[prior * tst + tid] = vc[tid];
  }
  extern __shared__ __align__(16) uint8_t staged_rows[];
  __nv_bfloat16* vs = reinterpret_cast<__nv_bfloat16*>(staged_rows);   // the tail's K rows first, then its V rows
  int staged = 0;
  if constexpr (LongTail) {
    staged = stage_tail_rows(vs, kt, tst, kc, prior, tail, StagedTailRows, tid, MergeThreads);
    stage_tail_wait();
    __syncthreads();
  }
  // tail scores for all heads of the group in one pass over the tail's K rows
  unit_tail_scores<LongTail ? RowsLong : RowsShort>(q + b * qsb + (int64_t)(kh * g) * qsh, qsh, g, kstat + (int64_t)unit * StatFloats, kt, tst, kc, prior, tail,
                             sm_log2, &ts[0][0], 1024, warp, MergeWarps, lane, vs, staged);
  if constexpr (LongTail) {
    __syncthreads();          // every warp has read its K rows
    stage_tail_rows(vs, vt, tst, vc, prior, tail, StagedTailRows, tid, MergeThreads);
  }
  grid_dependency_wait();     // the split pass has written all partials
  __shared__ int exchange_failed;
  if (xchg.world > 0) {
    // triples of this unit's next epoch from every rank that has tiles of it; bounded wait (1 s), then an error code
    const int epoch = xchg.seen[unit] + 1;
    if (tid == 0) exchange_failed = 0;
    __syncthreads();
    if (tid < xchg.world && xchg.present[(int64_t)tid * xchg.units + unit]) {
      const int32_t* flag = reinterpret_cast<const int32_t*>(xchg.local + exchange_flag_offset(xchg.world, xchg.rank_stride)) +
                            (int64_t)tid * xchg.units + unit;
      const uint64_t t0 = globaltimer_ns();
      while (load_acquire_sys(flag) < epoch) {
        if (globaltimer_ns() - t0 > 1000000000ull) { exchange_failed = 1; break; }
      }
    }
    __syncthreads();
    if (exchange_failed) {
      if (tid == 0) atomicCAS(err, ErrNone, ErrBarrierTimeout);
      if constexpr (LongTail) stage_tail_wait();   // no copy in flight when the CTA leaves
      return;
    }
    if (tid == 0) xchg.seen[unit] = epoch;
    const float* block = xchg.local + (int64_t)(epoch & 1) * xchg.world * xchg.rank_stride;
    const int64_t ug = (int64_t)xchg.units * MaxGroup;
    pm = block; pl = block + ug; po = block + 2 * ug;
  }
  if constexpr (LongTail) stage_tail_wait();
  __syncthreads();            // the tail scores of all warps (and the staged rows) are in shared memory; then warp r merges Q head r
  if (gather.world == 0) {
    if (warp < g)
      merge_head_by_warp<LongTail ? RowsLong : RowsShort>(pm, pl, po, (int64_t)sl.x * MaxGroup + warp, ml_stride, o_stride, sl.y, ts[warp], tail, prior, vt, tst, vc,
                                   vstat + (int64_t)unit * StatFloats, out + b * osb + (int64_t)(kh * g + warp) * osh, lane, vs, staged);
    return;
  }
  // unit sharding: the row is computed into shared memory once and stored into every GPU's full output tensor
  __shared__ __align__(16) __nv_bfloat16 rows[MaxGroup][D];
  const int epoch = gather.sync[1] + 1;          // read by every CTA before the last one to finish advances it
  if (warp < g)
    merge_head_by_warp<LongTail ? RowsLong : RowsShort>(pm, pl, po, (int64_t)sl.x * MaxGroup + warp, ml_stride, o_stride, sl.y, ts[warp], tail, prior, vt, tst, vc,
                                 vstat + (int64_t)unit * StatFloats, rows[warp], lane, vs, staged);
  __syncthreads();
  const int64_t row0 = (int64_t)(epoch & 1) * gather.rows_total + gather.unit_row[unit];
  for (int i = tid; i < gather.world * g * (D / 8); i += MergeThreads) {   // 16-byte pieces: peer, head row, piece
    const int p = i / (g * (D / 8)), r = (i / (D / 8)) % g, piece = i % (D / 8);
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(gather.peers[p]) + (row0 + r) * D + piece * 8;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&rows[r][piece * 8]);
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();                      // cumulative over the CTA's stores (the barrier made them visible here)
    const int done = atomicAdd(&gather.sync[0], 1);
    if (done == (int)gridDim.x - 1) {            // every CTA of the launch has stored and fenced
      gather.sync[0] = 0;
      gather.sync[1] = epoch;
      __threadfence_system();
      for (int p = 0; p < gather.world; ++p) {
        volatile int32_t* flags = reinterpret_cast<volatile int32_t*>(static_cast<char*>(gather.peers[p]) +
                                                                      gather_flag_offset_bytes(gather.rows_total));
        flags[gather.rank] = epoch;
      }
    }
  }
}

// Consumer of the output gather: one warp waits (at most one second, then device error 1) until every rank's flag has
// reached this GPU's next epoch; what follows in the stream sees the complete output of that step.
__global__ void __launch_bounds__(64) gather_wait_kernel(const void* local, int64_t rows_total, int32_t* seen, int world, int* err) {
  grid_dependency_wait();
  const int epoch = *seen + 1;
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const int32_t* flag = reinterpret_cast<const int32_t*>(static_cast<const char*>(local) + gather_flag_offset_bytes(rows_total)) + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    while (load_acquire_sys(flag) < epoch) {
      if (globaltimer_ns() - t0 > 1000000000ull) { failed = 1; break; }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (failed) atomicCAS(err, ErrNone, ErrBarrierTimeout);
    else *seen = epoch;
  }
}


// ---- cache store: gather kept tiles of the prefill operands into the per-unit streams ------------
// grid (max kept tiles, units), 256 threads.  K8 / V8 / V4 blobs are re-ordered from the prefill
// operand layout (tcgen05 core matrices, csrc/common.cuh) into the decode layout (decode_kernel.cuh):
// the same codes, permuted in 16-byte units (K8) or 32-bit words (V8, V4).  K4 blobs are already
// written in the decode layout.
__global__ void __launch_bounds__(256) cache_store_kernel(uint8_t* pool, const int64_t* unit_base, const int32_t* unit_tab,
    const int32_t* unit_count, const int32_t* unit_flags, const int2* tmeta, const uint8_t* k8, const uint8_t* k4,
    const float* ka, const float* ka4, const uint8_t* v8, const uint8_t* v4, int tiles) {
  const int i = blockIdx.x, unit = blockIdx.y, tid = threadIdx.x;
  if (i >= unit_count[unit] || (unit_flags[unit] & 1)) return;
  const int2 mt = tmeta[unit_tab[unit] + i];
  const uint32_t info = (uint32_t)mt.y;
  const int64_t ht = (int64_t)unit * tiles + (info & InfoTileMask);
  uint8_t* dst = pool + unit_base[unit] + (int64_t)mt.x * 16;
  const bool is_k4 = info & InfoK4, is_v4 = info & InfoV4;
  if (is_k4) {
    const uint4* src = reinterpret_cast<const uint4*>(k4 + ht * K4Bytes);
    for (int d = tid; d < K4Bytes / 16; d += 256) reinterpret_cast<uint4*>(dst)[d] = src[d];
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(k8 + ht * K8Bytes);
    for (int d = tid; d < K8Bytes / 16; d += 256) {
      const int blk = d / 64, h = (d % 64) / 32, key = (d % 32) / 4, sub = d % 4;
      reinterpret_cast<uint4*>(dst)[d] = src[blk * 64 + (2 * sub + h) * 8 + key];
    }
  }
  uint8_t* vd = dst + (is_k4 ? K4Bytes : K8Bytes);
  if (is_v4) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(v4 + ht * V4Bytes);
    for (int d = tid; d < V4Bytes / 8; d += 256) {      // one 8-byte run = (channel, sub): words kc = 0, 1
      const int cb = d / 32, ch = (d % 32) / 4, sub = d % 4;
      reinterpret_cast<uint2*>(vd)[d] = make_uint2(src[cb * 64 + ch * 4 + sub], src[cb * 64 + 32 + ch * 4 + sub]);
    }
  } else {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(v8 + ht * V8Bytes);
    for (int d = tid; d < V8Bytes / 16; d += 256) {     // one 16-byte run = (channel, sub): words of key groups 0..3
      const int cb = d / 32, ch = (d % 32) / 4, sub = d % 4;
      const uint32_t* s = src + cb * 128 + ch * 4 + sub;
      reinterpret_cast<uint4*>(vd)[d] = make_uint4(s[0], s[32], s[64], s[96]);
    }
  }
  if (tid == 0)
    *reinterpret_cast<uint4*>(vd + (is_v4 ? V4Bytes : V8Bytes)) = *reinterpret_cast<const uint4*>((is_k4 ? ka4 : ka) + ht * 4);
}

// grid (32-key chunks, listed BF16 units), 256 threads: K/V bf16 [B,Hkv,T,128] -> decode-layout chunks.
__global__ void __launch_bounds__(256) cache_store_bf16_kernel(uint8_t* pool, const int64_t* unit_base, const int32_t* units,
    const __nv_bfloat16* k, const __nv_bfloat16* v, int tokens, int heads, int64_t ksb, int64_t ksh, int64_t kst, int64_t vsb,
    int64_t vsh, int64_t vst, int chunk_begin) {
  const int unit = units[blockIdx.y];
  const __nv_bfloat16* kb = k + (unit / heads) * ksb + (unit % heads) * ksh;
  const __nv_bfloat16* vb = v + (unit / heads) * vsb + (unit % heads) * vsh;
  uint8_t* dst = pool + unit_base[unit] + (int64_t)blockIdx.x * Bf16ChunkBytes;   // the stream holds chunks begin, begin+1, ...
  const int key0 = (chunk_begin + blockIdx.x) * Bf16ChunkKeys;
  for (int d = threadIdx.x; d < 512; d += 256) {      // K: 16-byte runs [key/8][u][key%8][sub] = features 32sub+8u..+7
    const int nb = d / 128, u = (d % 128) / 32, key = key0 + nb * 8 + (d % 32) / 4, sub = d % 4;
    reinterpret_cast<uint4*>(dst)[d] = key < tokens ? *reinterpret_cast<const uint4*>(kb + (int64_t)key * kst + sub * 32 + u * 8)
                                                    : make_uint4(0, 0, 0, 0);
  }
  uint32_t* vd = reinterpret_cast<uint32_t*>(dst + 8192);
  for (int w = threadIdx.x; w < 2048; w += 256) {     // V words [ch/8][ch%8][sub][2ks+h] = keys 16ks+8h+2sub+{0,1}
    const int cb = w / 128, ch = cb * 8 + (w % 128) / 16, sub = (w % 16) / 4, ks = (w % 4) / 2, h = w % 2;
    const int key = key0 + ks * 16 + h * 8 + sub * 2;
    const uint32_t lo = key < tokens ? __bfloat16_as_ushort(vb[(int64_t)key * vst + ch]) : 0u;
    const uint32_t hi = key + 1 < tokens ? __bfloat16_as_ushort(vb[(int64_t)(key + 1) * vst + ch]) : 0u;
    vd[w] = lo | (hi << 16);
  }
}

static int configure_decode() {
  static TriPerDevice configured;   // the attribute belongs to the (function, device) pair
  const int device = configured.pending();
  TRI_CHECK(device != -2, "decode: no current CUDA device");
  if (device >= 0) {
    TRI_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeShared), "decode");
    TRI_CUDA(cudaFuncSetAttribute(decode_merge_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, StagedTailBytes), "decode");
    configured.mark(device);
  }
  return TRI_OK;
}

}  // namespace tri

using namespace tri;

extern "C" int tri_decode_occupancy(void) {
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  int blocks = 0;
  TRI_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, decode_kernel, DecodeThreads, DecodeShared), "decode_occupancy");
  return blocks;
}

namespace tri {
// Arguments shared by the decode entry points, after validation.
struct DecodeCall {
  const __nv_bfloat16* q; int64_t qsb, qsh;
  const uint8_t* pool; const int64_t* unit_base; const int32_t* unit_tab; const int32_t* unit_flags; const int2* tmeta;
  const int4* segments; const int32_t* cta_segments; int num_ctas; const int2* unit_slots;
  const float* kstat; const float* vstat; __nv_bfloat16* tail_k; __nv_bfloat16* tail_v; int64_t tsu, tst;
  const __nv_bfloat16* kcur; const __nv_bfloat16* vcur; int64_t csb, csh; const int64_t* step;
  __nv_bfloat16* out; int64_t osb, osh; int batch, heads_q, heads_kv, prompt, max_tail; float sm_log2; int* err;
};

static cudaError_t launch_split(const DecodeCall& c, float* pm, float* pl, float* po, int slot_limit, int stream_only,
                                const MergeArgs& margs, cudaStream_t s, bool chained) {
  if (chained)
    return launch_chained(decode_kernel, dim3(c.num_ctas), dim3(DecodeThreads), DecodeShared, s, c.q, c.qsb, c.qsh, c.pool,
                          c.unit_base, c.unit_tab, c.unit_flags, c.tmeta, c.segments, c.cta_segments, pm, pl, po, c.heads_q,
                          c.heads_kv, c.prompt, c.sm_log2, stream_only, slot_limit, margs, c.err);
  decode_kernel<<<c.num_ctas, DecodeThreads, DecodeShared, s>>>(c.q, c.qsb, c.qsh, c.pool, c.unit_base, c.unit_tab, c.unit_flags,
      c.tmeta, c.segments, c.cta_segments, pm, pl, po, c.heads_q, c.heads_kv, c.prompt, c.sm_log2, stream_only, slot_limit, margs,
      c.err);
  return cudaSuccess;
}

// How many rows the caller expects the BF16 tails to hold in the launches that follow on this host thread (a hint: it
// picks between two instantiations of the merge kernel that compute the same bits).  Negative = not known: the
// instantiation that is good at every length.
static thread_local int g_tail_hint = -1;
constexpr int LongTailRows = 8;

extern "C" int tri_decode_tail_hint(int rows) {
  g_tail_hint = rows;
  return TRI_OK;
}

template <bool LongTail>
static cudaError_t launch_merge_as(const DecodeCall& c, const float* pm, const float* pl, const float* po, int64_t ml_stride,
                                   int64_t o_stride, const int2* unit_slots, int slot_limit, cudaStream_t s, bool chained,
                                   SplitExchange xchg, OutputGather gather) {
  const dim3 grid(c.batch * c.heads_kv);
  if (chained)
    return launch_chained(decode_merge_kernel<LongTail>, grid, dim3(MergeThreads), LongTail ? StagedTailBytes : 0, s, pm, pl, po, ml_stride, o_stride, xchg, gather,
                          unit_slots, slot_limit, c.vstat, c.kstat, c.q, c.qsb, c.qsh, c.tail_k, c.tail_v, c.tsu, c.tst, c.kcur, c.vcur,
                          c.csb, c.csh, c.step, c.out, c.osb, c.osh, c.heads_q, c.heads_kv, c.max_tail, c.sm_log2, c.err);
  decode_merge_kernel<LongTail><<<grid, MergeThreads, LongTail ? StagedTailBytes : 0, s>>>(pm, pl, po, ml_stride, o_stride, xchg, gather, unit_slots, slot_limit, c.vstat,
      c.kstat, c.q, c.qsb, c.qsh, c.tail_k, c.tail_v, c.tsu, c.tst, c.kcur, c.vcur, c.csb, c.csh, c.step, c.out, c.osb, c.osh, c.heads_q,
      c.heads_kv, c.max_tail, c.sm_log2, c.err);
  return cudaSuccess;
}
static cudaError_t launch_merge(const DecodeCall& c, const float* pm, const float* pl, const float* po, int64_t ml_stride,
                                int64_t o_stride, const int2* unit_slots, int slot_limit, cudaStream_t s, bool chained,
                                SplitExchange xchg = SplitExchange{}, OutputGather gather = OutputGather{}) {
  return g_tail_hint < 0 || g_tail_hint > LongTailRows
             ? launch_merge_as<true>(c, pm, pl, po, ml_stride, o_stride, unit_slots, slot_limit, s, chained, xchg, gather)
             : launch_merge_as<false>(c, pm, pl, po, ml_stride, o_stride, unit_slots, slot_limit, s, chained, xchg, gather);
}

static MergeArgs fused_merge_args(const DecodeCall& c, int32_t* unit_done) {
  MergeArgs m{};
  m.unit_slots = c.unit_slots; m.unit_done = unit_done; m.vstat = c.vstat; m.kstat = c.kstat; m.ktail = c.tail_k;
  m.vtail = c.tail_v; m.tsu = c.tsu; m.tst = c.tst; m.kcur = c.kcur; m.vcur = c.vcur; m.csb = c.csb; m.csh = c.csh;
  m.step = c.step; m.out = c.out; m.osb = c.osb; m.osh = c.osh; m.max_tail = c.max_tail;
  return m;
}
constexpr int NoSlotLimit = 0x7fffffff;   // caller-allocated partials: their size is the caller's contract
}  // namespace tri

// Validation common to tri_decode, tri_decode_partials, tri_decode_merge and tri_decode_static.
#define TRI_DECODE_COMMON_CHECKS(name)                                                                                       \
  TRI_CHECK(q && unit_slots && kstat && vstat && tail_k && tail_v && kcur && vcur && step && out && device_error,           \
            name ": null buffers");                                                                                          \
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && heads_q / heads_kv <= MaxGroup &&         \
            max_tail >= 1 && max_tail <= 1024 && prompt > 0, "decode geometry/buffers");                                     \
  TRI_CHECK((reinterpret_cast<uintptr_t>(q) & 7u) == 0 && q_stride_b % 4 == 0 && q_stride_h % 4 == 0 &&                     \
            (reinterpret_cast<uintptr_t>(kcur) & 7u) == 0 && (reinterpret_cast<uintptr_t>(vcur) & 7u) == 0 &&               \
            cur_stride_b % 4 == 0 && cur_stride_h % 4 == 0 && (reinterpret_cast<uintptr_t>(tail_k) & 7u) == 0 &&            \
            (reinterpret_cast<uintptr_t>(tail_v) & 7u) == 0 && tail_stride_u % 4 == 0 && tail_stride_t % 4 == 0 &&          \
            (reinterpret_cast<uintptr_t>(out) & 7u) == 0 && out_stride_b % 4 == 0 && out_stride_h % 4 == 0 &&               \
            aligned16(vstat) && aligned16(kstat), name ": alignment (rows of q, kcur, vcur, the tails and out 8-byte aligned)")

#define TRI_DECODE_CALL()                                                                                                    \
  DecodeCall{static_cast<const __nv_bfloat16*>(q), q_stride_b, q_stride_h, static_cast<const uint8_t*>(pool), unit_base,    \
             unit_tab, unit_flags, reinterpret_cast<const int2*>(tmeta), reinterpret_cast<const int4*>(segments),           \
             cta_segments, num_ctas, reinterpret_cast<const int2*>(unit_slots), kstat, vstat,                               \
             static_cast<__nv_bfloat16*>(tail_k), static_cast<__nv_bfloat16*>(tail_v), tail_stride_u, tail_stride_t,        \
             static_cast<const __nv_bfloat16*>(kcur), static_cast<const __nv_bfloat16*>(vcur), cur_stride_b, cur_stride_h,  \
             step, static_cast<__nv_bfloat16*>(out), out_stride_b, out_stride_h, batch, heads_q, heads_kv, prompt, max_tail, \
             (float)(scale * 1.4426950408889634), device_error}

extern "C" int tri_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool, const int64_t* unit_base,
    const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments, const int32_t* cta_segments,
    int num_ctas, const int32_t* unit_slots, const float* kstat, const float* vstat, void* tail_k, void* tail_v,
    int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur, int64_t cur_stride_b,
    int64_t cur_stride_h, const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h, float* pm, float* pl,
    float* po, int32_t* unit_done, int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale, int phases,
    int* device_error, void* stream) {
  TRI_DECODE_COMMON_CHECKS("decode");
  TRI_CHECK(pool && unit_base && unit_tab && unit_flags && tmeta && segments && cta_segments && pm && pl && po && num_ctas >= 0,
            "decode: null buffers");
  TRI_CHECK(aligned16(pool) && aligned16(po), "decode: alignment");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const DecodeCall call = TRI_DECODE_CALL();
  // One launch when both phases are wanted and the caller provides the per-unit completion counters: the CTA
  // that finishes a unit's last segment merges it.  Otherwise the split pass and the merge are two launches.
  const bool fused = phases == 3 && unit_done != nullptr && num_ctas > 0;
  const MergeArgs margs = fused ? fused_merge_args(call, unit_done) : MergeArgs{};
  if (num_ctas > 0 && (phases & 1))
    TRI_CUDA(launch_split(call, pm, pl, po, NoSlotLimit, (phases & 4) ? 1 : 0, margs, s, true), "decode");
  if ((phases & 2) && !fused)
    TRI_CUDA(launch_merge(call, pm, pl, po, MaxGroup, (int64_t)MaxGroup * D, call.unit_slots, NoSlotLimit, s, true), "decode");
  return tri_launch_status("decode");
}

extern "C" int tri_decode_partials(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool,
    const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments,
    const int32_t* cta_segments, int num_ctas, const int32_t* unit_slots, float* pm, float* pl, float* po, int32_t* unit_done,
    float* fold_m, float* fold_l, float* fold_o, void* const* peer_buffers, int world, int rank, int32_t* epoch,
    int batch, int heads_q, int heads_kv, int prompt, double scale, int* device_error, void* stream) {
  TRI_CHECK(q && pool && unit_base && unit_tab && unit_flags && tmeta && segments && cta_segments && unit_slots && pm && pl &&
            po && unit_done && device_error, "decode_partials: null buffers");
  TRI_CHECK((peer_buffers != nullptr) != (fold_m != nullptr) && (fold_m != nullptr) == (fold_l != nullptr) &&
            (fold_m != nullptr) == (fold_o != nullptr),
            "decode_partials: either the fold buffers or the peers' exchange buffers");
  TRI_CHECK(peer_buffers == nullptr || (epoch != nullptr && world >= 1 && world <= 64 && rank >= 0 && rank < world),
            "decode_partials: exchange group");
  TRI_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0 && heads_q / heads_kv <= MaxGroup && prompt > 0 &&
            num_ctas >= 0, "decode geometry/buffers");
  TRI_CHECK(aligned16(pool) && aligned16(po) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && q_stride_b % 4 == 0 &&
            q_stride_h % 4 == 0, "decode_partials: alignment");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  if (num_ctas == 0) return TRI_OK;
  DecodeCall call{};
  call.q = static_cast<const __nv_bfloat16*>(q); call.qsb = q_stride_b; call.qsh = q_stride_h;
  call.pool = static_cast<const uint8_t*>(pool); call.unit_base = unit_base; call.unit_tab = unit_tab; call.unit_flags = unit_flags;
  call.tmeta = reinterpret_cast<const int2*>(tmeta); call.segments = reinterpret_cast<const int4*>(segments);
  call.cta_segments = cta_segments; call.num_ctas = num_ctas; call.unit_slots = reinterpret_cast<const int2*>(unit_slots);
  call.batch = batch; call.heads_q = heads_q; call.heads_kv = heads_kv; call.prompt = prompt;
  call.sm_log2 = (float)(scale * 1.4426950408889634); call.err = device_error;
  MergeArgs margs{};
  margs.unit_slots = call.unit_slots; margs.unit_done = unit_done; margs.fold_m = fold_m; margs.fold_l = fold_l; margs.fold_o = fold_o;
  if (peer_buffers != nullptr) {
    margs.peers = reinterpret_cast<float* const*>(peer_buffers); margs.world = world; margs.rank = rank;
    margs.units = batch * heads_kv; margs.rank_stride = (int64_t)batch * heads_kv * MaxGroup * (D + 2); margs.epoch = epoch;
  }
  TRI_CUDA(launch_split(call, pm, pl, po, NoSlotLimit, 0, margs, static_cast<cudaStream_t>(stream), true), "decode_partials");
  return tri_launch_status("decode_partials");
}

extern "C" int tri_decode_split(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool, const int64_t* unit_base,
    const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments, const int32_t* cta_segments,
    int num_ctas, const int32_t* unit_slots, const float* kstat, const float* vstat, void* tail_k, void* tail_v,
    int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur, int64_t cur_stride_b,
    int64_t cur_stride_h, const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h, float* pm, float* pl,
    float* po, int32_t* unit_done, void* const* peer_buffers, int world, int rank, int32_t* epoch, const int32_t* present,
    int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale, int* device_error, void* stream) {
  TRI_DECODE_COMMON_CHECKS("decode_split");
  TRI_CHECK(pool && unit_base && unit_tab && unit_flags && tmeta && segments && cta_segments && pm && pl && po && unit_done &&
            peer_buffers && epoch && present && num_ctas > 0, "decode_split: null buffers");
  TRI_CHECK(aligned16(pool) && aligned16(po) && world >= 1 && world <= 64 && rank >= 0 && rank < world, "decode_split: exchange group");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  const DecodeCall call = TRI_DECODE_CALL();
  MergeArgs margs = fused_merge_args(call, unit_done);
  margs.peers = reinterpret_cast<float* const*>(peer_buffers); margs.world = world; margs.rank = rank;
  margs.units = batch * heads_kv; margs.rank_stride = (int64_t)batch * heads_kv * MaxGroup * (D + 2); margs.epoch = epoch;
  margs.present = present;
  TRI_CUDA(launch_split(call, pm, pl, po, NoSlotLimit, 0, margs, static_cast<cudaStream_t>(stream), true), "decode_split");
  return tri_launch_status("decode_split");
}

extern "C" int tri_decode_merge(const void* q, int64_t q_stride_b, int64_t q_stride_h, const float* pm, const float* pl,
    const float* po, int64_t split_stride, const void* exchange_buffer, const int32_t* present, int32_t* seen, int world,
    void* const* gather_peers, int gather_world, int gather_rank, const int64_t* unit_row, int64_t rows_total, int32_t* gather_sync,
    const int32_t* unit_slots, const float* kstat, const float* vstat, void* tail_k,
    void* tail_v, int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur, int64_t cur_stride_b,
    int64_t cur_stride_h, const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h, int batch, int heads_q,
    int heads_kv, int max_tail, double scale, int* device_error, void* stream) {
  const int prompt = 1;
  TRI_DECODE_COMMON_CHECKS("decode_merge");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  SplitExchange xchg{};
  if (exchange_buffer != nullptr) {
    TRI_CHECK(present && seen && world >= 1 && world <= 64 && aligned16(exchange_buffer), "decode_merge: exchange group");
    xchg = SplitExchange{static_cast<const float*>(exchange_buffer), present, seen, world, batch * heads_kv,
                         (int64_t)batch * heads_kv * MaxGroup * (D + 2)};
    split_stride = xchg.rank_stride;
    pm = pl = po = static_cast<const float*>(exchange_buffer);   // replaced per unit by the epoch's parity block
  }
  TRI_CHECK(pm && pl && po && aligned16(po) && split_stride >= 0 && split_stride % 4 == 0, "decode_merge: partials");
  DecodeCall call{};
  call.q = static_cast<const __nv_bfloat16*>(q); call.qsb = q_stride_b; call.qsh = q_stride_h;
  call.kstat = kstat; call.vstat = vstat; call.tail_k = static_cast<__nv_bfloat16*>(tail_k); call.tail_v = static_cast<__nv_bfloat16*>(tail_v);
  call.tsu = tail_stride_u; call.tst = tail_stride_t; call.kcur = static_cast<const __nv_bfloat16*>(kcur);
  call.vcur = static_cast<const __nv_bfloat16*>(vcur); call.csb = cur_stride_b; call.csh = cur_stride_h; call.step = step;
  call.out = static_cast<__nv_bfloat16*>(out); call.osb = out_stride_b; call.osh = out_stride_h; call.batch = batch;
  call.heads_q = heads_q; call.heads_kv = heads_kv; call.max_tail = max_tail; call.sm_log2 = (float)(scale * 1.4426950408889634);
  call.err = device_error;
  OutputGather gather{};
  if (gather_peers != nullptr) {
    TRI_CHECK(unit_row && gather_sync && gather_world >= 1 && gather_world <= 64 && gather_rank >= 0 && gather_rank < gather_world &&
              rows_total > 0, "decode_merge: output gather group");
    gather = OutputGather{gather_peers, unit_row, gather_sync, gather_world, gather_rank, rows_total};
  }
  const int64_t ml = split_stride ? split_stride : MaxGroup, os = split_stride ? split_stride : (int64_t)MaxGroup * D;
  TRI_CUDA(launch_merge(call, pm, pl, po, ml, os, reinterpret_cast<const int2*>(unit_slots), NoSlotLimit,
                        static_cast<cudaStream_t>(stream), true, xchg, gather), "decode_merge");
  return tri_launch_status("decode_merge");
}

extern "C" int tri_gather_wait(const void* gather_buffer, int64_t rows_total, int32_t* seen, int world, int* device_error,
                               void* stream) {
  TRI_CHECK(gather_buffer && seen && device_error && world >= 1 && world <= 64 && rows_total > 0, "gather_wait: arguments");
  TRI_CUDA(launch_chained(gather_wait_kernel, dim3(1), dim3(64), 0, static_cast<cudaStream_t>(stream), gather_buffer, rows_total, seen,
                          world, device_error), "gather_wait");
  return tri_launch_status("gather_wait");
}

extern "C" int tri_cache_store(void* pool, const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_count,
    const int32_t* unit_flags, const int32_t* tmeta, int units, int max_count, const void* k8, const void* k4, const float* ka,
    const float* ka4, const void* v8, const void* v4, int tiles, void* stream) {
  TRI_CHECK(pool && unit_base && unit_tab && unit_count && unit_flags && tmeta && k8 && ka && v8, "cache_store: null buffers");
  TRI_CHECK(units > 0 && max_count > 0 && tiles > 0 && aligned16(pool) && aligned16(k8) && aligned16(k4) && aligned16(v8) &&
            aligned16(v4) && aligned16(ka) && aligned16(ka4), "cache_store: geometry/alignment");
  cache_store_kernel<<<dim3(max_count, units), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(pool),
      unit_base, unit_tab, unit_count, unit_flags, reinterpret_cast<const int2*>(tmeta), static_cast<const uint8_t*>(k8),
      static_cast<const uint8_t*>(k4), ka, ka4, static_cast<const uint8_t*>(v8), static_cast<const uint8_t*>(v4), tiles);
  return tri_launch_status("cache_store");
}

extern "C" int tri_cache_store_bf16(void* pool, const int64_t* unit_base, const int32_t* units, int num_units, const void* k,
    const void* v, int tokens, int heads_kv, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t, int64_t v_stride_b,
    int64_t v_stride_h, int64_t v_stride_t, int chunk_begin, int chunk_count, void* stream) {
  TRI_CHECK(pool && unit_base && units && k && v && num_units > 0 && tokens > 0 && heads_kv > 0, "cache_store_bf16: arguments");
  TRI_CHECK(k_stride_t % 8 == 0 && k_stride_h % 8 == 0 && k_stride_b % 8 == 0 && aligned16(k) && aligned16(pool),
            "cache_store_bf16: K rows must be 16-byte aligned");
  const int chunks = (tokens + Bf16ChunkKeys - 1) / Bf16ChunkKeys;
  TRI_CHECK(chunk_begin >= 0 && chunk_count > 0 && chunk_begin + chunk_count <= chunks, "cache_store_bf16: chunk range");
  cache_store_bf16_kernel<<<dim3(chunk_count, num_units), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(pool),
      unit_base, units, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), tokens, heads_kv,
      k_stride_b, k_stride_h, k_stride_t, v_stride_b, v_stride_h, v_stride_t, chunk_begin);
  return tri_launch_status("cache_store_bf16");
}

// ---- fold: one (m, l, o) per unit and Q head from the unit's segment partials ---------------------
// Used when a unit's tile range is split across GPUs: every rank folds its local segments, the
// folded triples (1,040 B per Q head) are all-gathered, and the merge kernel then sees one "segment" per
// rank.  Same arithmetic as the first half of decode_merge_kernel; no V de-normalisation, no tail.
namespace tri {
__global__ void __launch_bounds__(D) decode_fold_kernel(const float* pm, const float* pl, const float* po,
    const int2* unit_slots, float* fm, float* fl, float* fo, int group) {
  const int unit = blockIdx.x, ch = threadIdx.x;
  const int2 sl = unit_slots[unit];
  for (int r = 0; r < group; ++r) {
    float big = -FLT_MAX;
    for (int s = 0; s < sl.y; ++s) big = fmaxf(big, pm[(int64_t)(sl.x + s) * MaxGroup + r]);
    float o = 0.f, l = 0.f;
    for (int s = 0; s < sl.y; ++s) {
      const int64_t idx = (int64_t)(sl.x + s) * MaxGroup + r;
      const float w = exp2f(pm[idx] - big);
      o = fmaf(po[idx * D + ch], w, o);
      l = fmaf(pl[idx], w, l);
    }
    const int64_t dst = (int64_t)unit * MaxGroup + r;
    fo[dst * D + ch] = o;
    if (ch == 0) { fm[dst] = big; fl[dst] = l; }
  }
}
}  // namespace tri

extern "C" int tri_decode_fold(const float* pm, const float* pl, const float* po, const int32_t* unit_slots, float* fm,
    float* fl, float* fo, int units, int group, void* stream) {
  TRI_CHECK(pm && pl && po && unit_slots && fm && fl && fo, "decode_fold: null buffers");
  TRI_CHECK(units > 0 && group >= 1 && group <= MaxGroup, "decode_fold: geometry");
  decode_fold_kernel<<<units, D, 0, static_cast<cudaStream_t>(stream)>>>(pm, pl, po, reinterpret_cast<const int2*>(unit_slots),
      fm, fl, fo, group);
  return tri_launch_status("decode_fold");
}

// ---- decode step for callers that cannot allocate device memory -----------------------------------
// Some callers of this library own no allocator on the GPU: a serving runtime that has handed every
// byte of HBM to its paged KV pool before the first request arrives, or a host language binding that
// can pass tensors it was given but has no way to ask the driver for more.  tri_decode needs scratch
// for the split-KV partials (pm, pl, po); this variant keeps that scratch inside the library image, in
// a fixed array that every GPU loading the library holds until the process exits.
constexpr int StaticSlots = 1024;                                     // partial slots (segments) per call, at most
constexpr size_t StaticFloats = (size_t)StaticSlots * MaxGroup * (D + 2);
static __device__ __align__(256) float g_static_partials[StaticFloats];   // 4,259,840 bytes per GPU

// Device address of the array, looked up once per device.  In host code the array's name is only a
// handle for the runtime, never an address a kernel may use.
static float* static_partials_for_current_device(void) {
  constexpr int MaxDevices = 64;
  static float* known[MaxDevices] = {};
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MaxDevices) return nullptr;
  if (known[device] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_partials) != cudaSuccess) return nullptr;
    known[device] = static_cast<float*>(p);
  }
  return known[device];
}

extern "C" int tri_decode_static(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool,
    const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments,
    const int32_t* cta_segments, int num_ctas, int num_slots, const int32_t* unit_slots, const float* kstat, const float* vstat,
    void* tail_k, void* tail_v, int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur,
    int64_t cur_stride_b, int64_t cur_stride_h, const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h,
    int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale, int* device_error, void* stream) {
  TRI_DECODE_COMMON_CHECKS("decode_static");
  TRI_CHECK(pool && unit_base && unit_tab && unit_flags && tmeta && segments && cta_segments && num_ctas > 0 && num_slots > 0 &&
            aligned16(pool), "decode_static: null buffers");
  TRI_CHECK(num_slots <= StaticSlots,
            "decode_static: more than 1024 partial slots (segments); use tri_decode with caller-allocated partials");
  if (configure_decode() != TRI_OK) return TRI_ERR_CUDA;
  float* scratch = static_partials_for_current_device();
  if (scratch == nullptr) {
    tri_set_error("decode_static: cudaGetSymbolAddress failed for the partials array on the current device");
    return TRI_ERR_CUDA;
  }
  // Nothing in the array has to start at zero: the split pass writes every (slot, Q head) entry that the
  // merge reads, so the previous call's contents are simply overwritten.  Both kernels get the array's capacity:
  // a slot number at or beyond it (a plan whose slot column is not 0 .. num_slots-1) is not stored to or read
  // from; the kernel records ErrBadSlot in the device error word instead.
  float* pm = scratch;
  float* pl = scratch + (size_t)StaticSlots * MaxGroup;
  float* po = scratch + (size_t)StaticSlots * MaxGroup * 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const DecodeCall call = TRI_DECODE_CALL();
  TRI_CUDA(launch_split(call, pm, pl, po, StaticSlots, 0, MergeArgs{}, s, false), "decode_static");
  TRI_CUDA(launch_merge(call, pm, pl, po, MaxGroup, (int64_t)MaxGroup * D, call.unit_slots, StaticSlots, s, false), "decode_static");
  return tri_launch_status("decode_static");
}
