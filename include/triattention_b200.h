/* C ABI of libtriattn_sm100a.so — the B200 (sm_100a) kernels behind TriAttention's quantised
 * attention path.  Plain pointers and sizes only; every pointer is a device pointer unless it says
 * "host".  All functions return 0 on success or a negative status and leave a message for
 * tri_last_error().  Work is enqueued on `stream` (a cudaStream_t); nothing synchronises the host.
 * The caller allocates every buffer, like the reference's callers do
 * (triattention/kernels/prefill.py:42-85, triattention/kernels/decode.py:62-75).
 *
 * "Replaces" lines name the reference interface each entry point stands in for (paths inside the
 * reference project).  The reference is batch 1 everywhere; these take a batch count, and
 * unit = sequence * heads + head indexes the leading dimension of every per-head buffer.
 *
 * Tile blob layouts (K8, K4X, K4, V8, V4, V16) are documented in triattention_b200/csrc/common.cuh.
 */
#ifndef TRIATTENTION_B200_H
#define TRIATTENTION_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { TRI_OK = 0, TRI_ERR_ARGUMENT = -1, TRI_ERR_CUDA = -2, TRI_ERR_DEVICE = -3 };
/* Values of the device error word (`device_error` arguments): 1 = a bounded barrier wait ran out, 3 = a tile number
 * outside the prompt in a task table, 4 = a partial slot outside the partial buffers. */

/* Message of the last failing call made by this host thread. */
const char* tri_last_error(void);
int tri_abi_version(void);

/* Rotate + quantise Q (per token) and K (centred by the channel mean over the prompt, per 16-key
 * group) into tensor-core operands.
 * Replaces prepare_qk(q,k,q8,qa,kp,ka,partial,kstat,q4,qa4,k4p,ka4),
 *   triattention/kernels/cuda/common_host.cuh:1-25.
 * q  bf16 [B,Hq,T,128], k bf16 [B,Hkv,T,128]: element strides given, feature stride 1, rows 16-byte aligned.
 * q8 int8 [B*Hq,T,128]; qa f32 [B*Hq,T]; k8 K8 blobs [B*Hkv,tiles,8192 B]; ka f32 [B*Hkv,tiles,4];
 * partial f32 [B*Hkv,64,3,128] scratch; kstat f32 [B*Hkv,3,128] (mean, -, -).
 * INT4 outputs, all or none: q4x int8 [B*Hq,T,128] (4-bit codes as int8), qa4, k4x K4X blobs
 * [B*Hkv,tiles,8192 B], ka4; k4 (optional with the others) packed K4 blobs [B*Hkv,tiles,4096 B].
 * q_modes int32 [Hq] on the device or NULL (no counterpart in the reference, which quantises every head both ways):
 * what tri_attention will read of each Q head, bit 0 = the INT8 codes, bit 1 = the INT4 codes; rows of q8 / q4x
 * (and qa / qa4) whose bit is clear are left untouched.  NULL = every head, both. */
int tri_prepare_qk(const void* q, const void* k, int batch, int heads_q, int heads_kv, int tokens,
                   int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                   int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                   void* q8, float* qa, void* k8, float* ka, float* partial, float* kstat,
                   void* q4x, float* qa4, void* k4x, void* k4, float* ka4, const int32_t* q_modes, void* stream);

/* Per-channel affine normalisation of V and packing into FP16 / INT8 / INT4 tile blobs.
 * Replaces pack_v(v,partial,vstat,v16p,v8p,v4p), triattention/kernels/cuda/common_host.cuh:27-45.
 * vstat f32 [B*Hkv,3,128] = (mean, scale, 1/scale); (0,1,1) when neither v8 nor v4 is requested.
 * v16 [B*Hkv,tiles,16384 B], v8 [..,8192 B], v4 [..,4096 B]; each may be NULL.
 * v8h [B*Hkv,tiles,16384 B] (may be NULL; no counterpart in the reference): the INT8 codes again as fp16 numbers
 * in the v16 layout, the P.V operand of tri_attention, whose tensor-core weights are fp16.
 * raw_heads int32 [Hkv] on the device or NULL (no counterpart in the reference): non-zero marks an un-quantised
 * (BF16) KV head; its units get identity statistics (0, 1, 1) and only the v16 blob, holding V itself as fp16
 * (values beyond +-65504 clamped), which is what tri_attention reads for such heads. */
int tri_pack_v(const void* v, int batch, int heads_kv, int tokens,
               int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
               float* partial, float* vstat, void* v16, void* v8, void* v4, void* v8h,
               const int32_t* raw_heads, void* stream);

/* tri_prepare_qk and tri_pack_v as ONE call (no counterpart in the reference, whose executor makes the two calls one
 * after the other, triattention/kernels/prefill.py:99-101): same arguments, same kernels and bit-identical results, but
 * the three independent chains — Q (one bandwidth-bound kernel), K (statistics, then codes) and V (statistics, then
 * blobs) — run side by side: Q on `stream`, K and V on two streams owned by the library that start behind everything
 * already queued on `stream` and that `stream` waits for before the call's results can be used.  partial_k and partial_v
 * are two scratch buffers of the size tri_prepare_qk / tri_pack_v document (they must differ).  Safe to call from
 * several host threads (calls on one device take turns for the time it takes to queue the launches). */
int tri_write_kv(const void* q, const void* k, const void* v, int batch, int heads_q, int heads_kv, int tokens,
                 int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                 int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                 int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
                 void* q8, float* qa, void* k8, float* ka, float* partial_k, float* kstat,
                 void* q4x, float* qa4, void* k4x, void* k4, float* ka4, const int32_t* q_modes,
                 float* partial_v, float* vstat, void* v16, void* v8, void* v4, void* v8h,
                 const int32_t* raw_heads, void* stream);

/* Quantise K and V rows that arrive after the prompt with the prompt's statistics (no statistics pass): K8 blobs
 * and scales as tri_prepare_qk writes them, V8 blobs as tri_pack_v writes them, rows >= tokens zero.  The decode cache
 * uses it to turn 64 generated tokens of the BF16 tail into one more cached tile (no counterpart in the reference,
 * whose tail is capped at 1024 tokens, triattention/kernels/cuda/common_host.cuh:56).
 * k, v bf16 [B,Hkv,T,128] with element strides; kstat, vstat f32 [B*Hkv,3,128] (read only);
 * k8 [B*Hkv,tiles,8192 B]; ka f32 [B*Hkv,tiles,4]; v8 [B*Hkv,tiles,8192 B]. */
int tri_requantize_kv(const void* k, const void* v, int batch, int heads_kv, int tokens,
                      int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                      int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
                      const float* kstat, const float* vstat, void* k8, float* ka, void* v8, void* stream);

/* Banded causal prefill attention (tcgen05).
 * Replaces attention(order,bands,groups,entries,v16p,v8p,v4p,vstat,q8,k8p,qa8,ka8,q4,k4p,qa4,ka4,out,scale),
 *   triattention/kernels/cuda/prefill_sm80.cu:510-543, in band mode.  The CTA order is internal
 *   (heaviest query blocks first); task-table mode (groups/entries) is tri_attention_tasks.
 * bands int32 [Hq,2] = (w8,w4) in tile distances.  out is bf16 (or fp16 when out_is_half) [B,Hq,T,128]
 * with element strides.  v8h: the fp16 rendering of the INT8 V codes from tri_pack_v (where the reference passes
 * its v8p).  device_error: int32 word, set non-zero if a bounded wait ran out.
 * Un-quantised (BF16) heads, an extension (the reference's only BF16 attention is torch's SDPA,
 * triattention/models.py:45-47): a head with w8 < 1 is computed by the same kernel as exact causal attention over
 * every tile — bf16 QK^T with fp32 scores and an exact online softmax on the tensor cores — from the caller's own
 * tensors q_raw bf16 [B,Hq,T,128] and k_raw bf16 [B,Hkv,T,128] (element strides, rows 16-byte aligned; read by TMA
 * tensor copies) and the v16 blobs that tri_pack_v wrote for a raw head.  With q_raw = k_raw = NULL such heads are
 * skipped. */
int tri_attention(const int32_t* bands, const void* v16, const void* v8h, const float* vstat,
                  const void* q8, const void* k8, const float* qa8, const float* ka8,
                  const void* q4x, const void* k4x, const float* qa4, const float* ka4,
                  void* out, int out_is_half, int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t,
                  int batch, int heads_q, int heads_kv, int tokens, double scale,
                  const void* q_raw, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                  const void* k_raw, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                  int* device_error, void* stream);

/* Several band maps over the same operands in ONE launch, and only the query rows that are wanted: what the reference's
 * calibration tool does with one full prefill per grid point (triattention/calibrate.py:46-63: ~90 (w8, w4)
 * configurations per layer and sample, each re-quantising Q, K, V and computing every row, of which it keeps the last
 * 1024).  bands int32 [configs, Hq, 2]; configuration c writes out + c * out_stride_c.  first_block: query blocks (64
 * rows) before it are not computed; because a CTA owns four query blocks, rows from (first_block / 4) * 256 on are
 * written, at out + row * out_stride_t as usual (pass the pointer of a row-0 origin; rows before that are never
 * touched).  Quantised heads only; other arguments as tri_attention. */
int tri_attention_sweep(const int32_t* bands, int configs, int first_block, const void* v16, const void* v8h,
                        const float* vstat, const void* q8, const void* k8, const float* qa8, const float* ka8,
                        const void* q4x, const void* k4x, const float* qa4, const float* ka4,
                        void* out, int out_is_half, int64_t out_stride_c, int64_t out_stride_b, int64_t out_stride_h,
                        int64_t out_stride_t, int batch, int heads_q, int heads_kv, int tokens, double scale,
                        int* device_error, void* stream);

/* Task-table mode of the prefill attention: every (Q head, query block) brings four explicit tile lists.
 * Replaces attention(order,None,groups,entries,...), triattention/kernels/cuda/prefill_sm80.cu:287-292,510-543
 *   (no caller in the reference; kept for interface completeness as a CUDA-core kernel, not a tensor-core one).
 * groups int32 [Hq*rows*4+1] = offsets into entries int32 [...] of tile numbers; block (h, qb) runs
 * entries[groups[i]..groups[i+1]) for i = (h*rows+qb)*4 + pass: pass 0 INT8 scores / fp16 weights / V16, pass 1 INT8
 * scores / 8-bit P / V8, pass 2 INT8 scores / 4-bit P / V4, pass 3 INT4 scores (q4x, k4x) / 8-bit P / V8.  Only the
 * last tile of a pass is masked, and only if it is the block's diagonal tile.  The tables are shared by the batch.
 * A tile number outside the prompt is skipped and recorded in device_error (3).  Other operands as tri_attention,
 * with the INT8 V blobs themselves (v8) instead of their fp16 rendering, plus v4. */
int tri_attention_tasks(const int32_t* groups, const int32_t* entries, const void* v16, const void* v8, const void* v4,
                        const float* vstat, const void* q8, const void* k8, const float* qa8, const float* ka8,
                        const void* q4x, const void* k4x, const float* qa4, const float* ka4, void* out, int out_is_half,
                        int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t, int batch, int heads_q,
                        int heads_kv, int tokens, double scale, int* device_error, void* stream);

/* Gather the kept tiles of the prefill operands into per-(sequence, KV head) cache streams.
 * Replaces the index_select gathers of DecodeCache.store, triattention/kernels/decode.py:46-61.
 * Stream of a quantised unit: per kept tile, ascending, one chunk = K blob (K8 8192 B or K4 4096 B),
 * V blob (V8 8192 B or V4 4096 B), 4 f32 K scales.  unit_base int64 [U] byte offsets into pool;
 * unit_tab int32 [U] first row of the unit's table in tmeta; unit_count int32 [U]; unit_flags int32
 * [U] (bit 0: BF16 unit, skipped here); tmeta int32 [N,2] = (chunk offset in 16-byte units from the
 * unit base, info) with info = tile | rowmask<<12 | K4<<20 | V4<<21 | BF16<<22. */
int tri_cache_store(void* pool, const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_count,
                    const int32_t* unit_flags, const int32_t* tmeta, int units, int max_count,
                    const void* k8, const void* k4, const float* ka, const float* ka4,
                    const void* v8, const void* v4, int tiles, void* stream);

/* Same for un-quantised BF16 units (an extension; the reference has no BF16 heads in its kernels):
 * K and V rows are copied into 32-key chunks of 16384 B in MMA fragment order.  units int32 [n].
 * Chunks chunk_begin .. chunk_begin+chunk_count-1 of each unit are written, starting at the unit's base
 * (the whole prompt, or this GPU's part of it when the sequence is split across GPUs). */
int tri_cache_store_bf16(void* pool, const int64_t* unit_base, const int32_t* units, int num_units,
                         const void* k, const void* v, int tokens, int heads_kv,
                         int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                         int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
                         int chunk_begin, int chunk_count, void* stream);

/* One decode step of one layer for the whole batch: split-KV pass over the cache streams, then the
 * merge with the BF16 tail of generated tokens (the current K/V row is appended to the tail).
 * Replaces decode(q,k8c,k4c,ka,ka4,entry,kinfo,count,fmt,slot,v8,v4,vstat,kstat,ktail,vtail,kcur,vcur,
 *   step,out,pm,pl,po,prompt,per,scale), triattention/kernels/cuda/common_host.cuh:47-87.
 * The split pass runs num_ctas persistent CTAs (one per SM); CTA c streams segments
 * cta_segments[c] .. cta_segments[c+1]-1 (int32 [num_ctas+1]) of segments int32 [S,4] =
 * (unit, first kept tile, tile count, partial slot): a cost-balanced contiguous cut of the tile sequence.
 * unit_slots int32 [U,2] = (first partial slot, number of splits); pm, pl f32 [P,8]; po f32 [P,8,128];
 * tail_k/tail_v bf16 [U,max_tail,128] with element strides; kcur/vcur bf16 [B,Hkv,1,128];
 * step int64 [1] on the device; out bf16 [B,Hq,1,128].  phases: 1 = split pass only, 2 = merge only,
 * 3 = both (normal use; the single phases exist so that each kernel can be timed alone); 5 = split pass
 * that only streams the cache through shared memory without arithmetic (diagnostic of the copy pipeline).
 * unit_done int32 [U], zero before the first call, or NULL.  With it and phases = 3 the step is ONE launch:
 * the CTA that finishes a unit's last segment merges that unit (every unit needs >= 1 segment); the
 * counters are left at zero again.  With NULL the split pass and the merge are two launches. */
int tri_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool, const int64_t* unit_base,
               const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments,
               const int32_t* cta_segments, int num_ctas, const int32_t* unit_slots, const float* kstat, const float* vstat, void* tail_k, void* tail_v,
               int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur,
               int64_t cur_stride_b, int64_t cur_stride_h, const int64_t* step, void* out,
               int64_t out_stride_b, int64_t out_stride_h, float* pm, float* pl, float* po, int32_t* unit_done,
               int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale, int phases,
               int* device_error, void* stream);

/* Fold a unit's segment partials into one (m, l, o) per Q head: fm, fl f32 [U,8], fo f32 [U,8,128].
 * Stand-alone form of the fold that tri_decode_partials does inside the split pass; kept for callers that
 * already hold segment partials.  Extends the split merge of
 * triattention/kernels/cuda/common_device.cuh:418-438 across devices; the reference is single-GPU. */
int tri_decode_fold(const float* pm, const float* pl, const float* po, const int32_t* unit_slots,
                    float* fm, float* fl, float* fo, int units, int group, void* stream);

/* Sequence split across GPUs, this GPU's part: the split pass of tri_decode over this rank's tiles, and in
 * the same launch the fold of every unit's segments to one (m, l, o) per Q head (the CTA that finishes a
 * unit's last segment folds it).  unit_done int32 [U], zero before the first call, left at zero.  The triples go
 *   - either into fold_m, fold_l f32 [U,8], fold_o f32 [U,8,128] for the caller to exchange (one NCCL all-gather);
 *     a unit without any segment on this rank is not touched: give its entries m = -FLT_MAX, l = 0, o = 0 once;
 *   - or (fold_* NULL, peer_buffers given) straight into the exchange buffer of every GPU of the group by peer stores,
 *     each followed by a flag: the compute step and the collective are one kernel.  peer_buffers: device array of
 *     `world` pointers, entry r = rank r's exchange buffer as mapped into THIS process (symmetric / peer memory; this
 *     rank's own buffer at entry `rank`).  Buffer layout, in 4-byte words: data f32 [2][world][U*8*130] (parity of the
 *     step's epoch, source rank, then m [U,8] | l [U,8] | o [U,8,128]) followed by flags int32 [world][U].  Before the
 *     first step every rank fills its own buffer with m = -FLT_MAX, l = 0, o = 0, flags = 0 and the group synchronises
 *     once.  epoch int32 [U], zero at first: the steps this rank has folded, per unit.  tri_decode_merge with
 *     `exchange_buffer` is the matching consumer.  Every GPU of the group must run the same sequence of steps.
 * No counterpart in the reference (single GPU). */
int tri_decode_partials(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool,
                        const int64_t* unit_base, const int32_t* unit_tab, const int32_t* unit_flags,
                        const int32_t* tmeta, const int32_t* segments, const int32_t* cta_segments, int num_ctas,
                        const int32_t* unit_slots, float* pm, float* pl, float* po, int32_t* unit_done,
                        float* fold_m, float* fold_l, float* fold_o,
                        void* const* peer_buffers, int world, int rank, int32_t* epoch,
                        int batch, int heads_q, int heads_kv, int prompt, double scale,
                        int* device_error, void* stream);

/* A whole decode step of a sequence-split group on this GPU as ONE kernel: the split pass over this rank's tiles, the
 * fold of every unit to one triple, its delivery into every GPU's exchange buffer by peer stores (as
 * tri_decode_partials with peer_buffers), and — in the CTA that delivered it — the wait for the other ranks' triples
 * of that unit (at most one second, then device error 1) and the merge with the BF16 tail into `out`.  Compute step and
 * collective are fused; no NCCL call and no second launch.  present int32 [world,U]: rank r holds tiles of unit u;
 * every rank must hold tiles of every unit (otherwise use tri_decode_partials + tri_decode_merge, which also merge
 * units this rank has no tiles of).  Other arguments as tri_decode / tri_decode_partials.
 * No counterpart in the reference (single GPU). */
int tri_decode_split(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool, const int64_t* unit_base,
                     const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments,
                     const int32_t* cta_segments, int num_ctas, const int32_t* unit_slots, const float* kstat,
                     const float* vstat, void* tail_k, void* tail_v, int64_t tail_stride_u, int64_t tail_stride_t,
                     const void* kcur, const void* vcur, int64_t cur_stride_b, int64_t cur_stride_h,
                     const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h,
                     float* pm, float* pl, float* po, int32_t* unit_done,
                     void* const* peer_buffers, int world, int rank, int32_t* epoch, const int32_t* present,
                     int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale,
                     int* device_error, void* stream);

/* The merge of tri_decode alone, over partials that may lie strided: split s of unit u is read at
 * pm[(first*8 + r) + s*split_stride], pl likewise, po[(first*8 + r)*128 + ch + s*split_stride] with
 * (first, count) = unit_slots[u].  split_stride = 0 means the dense buffers of the split pass.  With
 * triples all-gathered as [rank][m | l | o] and unit_slots[u] = (u, world), split_stride = the floats per rank:
 * the gathered buffer is merged in place, no re-layout.
 * exchange_buffer (or NULL): this rank's exchange buffer of the peer-memory exchange (tri_decode_partials); pm, pl, po
 * and split_stride are then ignored: the CTA of a unit waits — at most one second, then device error 1 — until every
 * source rank r with present[r*U + u] != 0 (int32 [world,U]: rank r holds tiles of unit u) has delivered the triple
 * of the unit's next epoch, and merges that epoch's block.  seen int32 [U], zero at first: the steps merged so far.
 * gather_peers (or NULL): output gather by peer stores, for units sharded across GPUs.  Instead of `out`, every Q-head
 * row is stored into the full output tensor of EVERY GPU of the group: gather_peers = device array of gather_world
 * pointers, entry r = rank r's gather buffer as mapped into this process, laid out as bf16 [2][rows_total][128] (parity
 * of the step, then the rows of the full [B, Hq] output) followed, 64-byte aligned, by int32 flags [gather_world], all
 * zero at first.  unit_row int64 [U]: row of this rank's unit u's first Q head in the full tensor.  gather_sync int32 [2],
 * zero at first (finished CTAs, steps done).  The last CTA to finish raises this rank's flag on every GPU;
 * tri_gather_wait is the consumer.  Every rank must run the same sequence of steps.
 * Other arguments as tri_decode.
 * Replaces decode_merge_kernel, triattention/kernels/cuda/common_device.cuh:373-469. */
int tri_decode_merge(const void* q, int64_t q_stride_b, int64_t q_stride_h, const float* pm, const float* pl,
                     const float* po, int64_t split_stride,
                     const void* exchange_buffer, const int32_t* present, int32_t* seen, int world,
                     void* const* gather_peers, int gather_world, int gather_rank, const int64_t* unit_row,
                     int64_t rows_total, int32_t* gather_sync,
                     const int32_t* unit_slots, const float* kstat,
                     const float* vstat, void* tail_k, void* tail_v, int64_t tail_stride_u, int64_t tail_stride_t,
                     const void* kcur, const void* vcur, int64_t cur_stride_b, int64_t cur_stride_h,
                     const int64_t* step, void* out, int64_t out_stride_b, int64_t out_stride_h,
                     int batch, int heads_q, int heads_kv, int max_tail, double scale,
                     int* device_error, void* stream);

/* Consumer of the output gather of tri_decode_merge: one small launch that waits (at most one second, then device error
 * 1) until the flag of every rank in this GPU's gather buffer has reached the next step, so that whatever follows in the
 * stream reads the complete output of the step from parity block (step & 1), counting steps from 1.  seen int32 [1],
 * zero at first.  No counterpart in the reference (single GPU). */
int tri_gather_wait(const void* gather_buffer, int64_t rows_total, int32_t* seen, int world, int* device_error, void* stream);

/* tri_decode for callers that cannot allocate device memory (a runtime that gave all of HBM to its KV
 * pool up front, a binding that can only pass buffers it was handed).  Same arguments as tri_decode
 * without pm / pl / po and without phases: the split-KV partials live in a fixed 4,259,840-byte array
 * inside the library, held by every GPU that loads it until the process exits.  num_slots = number of
 * rows of `segments`; more than 1024 is refused with TRI_ERR_ARGUMENT (use tri_decode then).  The slot
 * numbers in `segments[:,3]` and `unit_slots` must be 0 .. num_slots-1 (what a plan from plan_streams holds);
 * the kernels check every slot against the array's capacity and, for one outside it, store and read nothing
 * and set the device error word to 4.  A cudaDeviceReset invalidates the cached address.  The call
 * makes no allocation of any kind.  The first call on each device looks up the array's device address
 * (with that device current), so make that first call outside any stream capture.  All calls on a device
 * share the array: calls that can overlap on the GPU (different streams) race on it, so keep them on
 * one stream or order them yourself.  Nothing needs clearing between calls.
 * No counterpart in the reference, whose Python caller allocates the partials (kernels/decode.py:72-75). */
int tri_decode_static(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* pool, const int64_t* unit_base,
                      const int32_t* unit_tab, const int32_t* unit_flags, const int32_t* tmeta, const int32_t* segments,
                      const int32_t* cta_segments, int num_ctas, int num_slots, const int32_t* unit_slots,
                      const float* kstat, const float* vstat, void* tail_k, void* tail_v,
                      int64_t tail_stride_u, int64_t tail_stride_t, const void* kcur, const void* vcur,
                      int64_t cur_stride_b, int64_t cur_stride_h, const int64_t* step, void* out,
                      int64_t out_stride_b, int64_t out_stride_h,
                      int batch, int heads_q, int heads_kv, int prompt, int max_tail, double scale,
                      int* device_error, void* stream);

/* How many rows the BF16 tails hold in the decode launches that follow on this host thread (the token being appended
 * included); negative = not known, the state a thread starts in.  A hint: it picks between two instantiations of the
 * merge kernel with the same arithmetic in the same order (bit-equal results) for the separate merge launch of tri_decode
 * (unit_done NULL), tri_decode_static and tri_decode_merge.  Up to 8 rows the one whose row loops are not unrolled runs
 * (4 us per step less at one row, 120 us more at 256 rows); above 8 rows, or without a hint, the one that unrolls them
 * and copies the tail rows into 64 KB of dynamic shared memory first.  Under
 * stream capture the instantiation chosen at capture time is the one replayed.  No counterpart in the reference (one merge
 * kernel, triattention/kernels/cuda/decode.cu). */
int tri_decode_tail_hint(int rows);

/* Resident decode CTAs per SM.  Replaces decode_occupancy(), triattention/kernels/cuda/common_host.cuh:89-94. */
int tri_decode_occupancy(void);

/* Integer QK^T accumulators of chosen tiles through the prefill kernel's operand path (TMA + tcgen05),
 * for parity checks.  requests int32 [n,4] = (Q unit, query-block pair, key tile, 0 = INT8 / 1 = INT4 codes);
 * acc int32 [n,128,64].  No counterpart in the reference (its accumulators never leave registers). */
int tri_qk_accumulators(const int32_t* requests, int num_requests, const void* q8, const void* q4x, const void* k8,
                        const void* k4x, int32_t* acc, int batch, int heads_q, int heads_kv, int tokens,
                        int* device_error, void* stream);

#ifdef __cplusplus
}
#endif
#endif
