/* C ABI of the B200 (sm_100a) NF4 fused-dequant linear path.
 *
 * The first block of declarations is the interface deep-fold's Python side
 * binds for this path (reference: gpu/include/chr_gpu.h); struct layouts, entry
 * names, argument order and return codes are kept so that the reference's
 * binding layer can call this library unchanged. The second block is additive:
 * entries the reference does not have (batched GEMV, embedding row decode,
 * fused greedy pick). Nothing here takes or returns a framework type: plain
 * pointers, sizes and a cudaStream_t passed as void*.
 *
 * Ownership: the caller owns every buffer, including split-K and attention
 * workspaces. No entry point allocates device memory. Return codes, shared by
 * every int-returning entry (reference: gpu/include/chr_gpu.h:30-33):
 *    0 ok            -1 null pointer          -2 N out of range
 *   -3 bad dims or null packed/scale          -4 K_pad != 64*ceil(K/64)
 *   -5 alignment (packed and x 16 B, scale 2 B)
 *   -6 CUDA launch or attribute failure       -7 workspace too small
 */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* Interface kept from the reference                                         */
/* ------------------------------------------------------------------------ */

/* One NF4 group-64 matrix resident on the device. Field order is frozen
 * (reference: gpu/include/chr_gpu.h:11-17). Byte packed[r][c] holds W[r][2c] in
 * its low nibble and W[r][2c+1] in its high nibble; scale[r][g] covers columns
 * 64g..64g+63 of row r. Columns K..K_pad-1 exist in the blobs and are ignored. */
typedef struct {
  int32_t M;              /* logical out_features */
  int32_t K;              /* logical in_features */
  int32_t K_pad;          /* 64 * ceil(K / 64) */
  const uint8_t *packed;  /* device, [M, K_pad/2] row-major */
  const uint16_t *scale;  /* device, [M, K_pad/64], IEEE binary16 bits */
} chr_nf4_dev_t;

/* Launch description returned by chr_nf4_gemm_plan (reference:
 * gpu/include/chr_gpu.h:48-61; same fields, sm_100a tile values). */
typedef struct {
  int32_t path;            /* 0 tcgen05 tile, BN from N; see CHR_PATH_* below */
  int32_t grid_x;          /* ceil(M / bm) */
  int32_t grid_y;          /* split_k */
  int32_t block;           /* threads per CTA */
  int32_t bm;              /* rows of M per CTA */
  int32_t bk;              /* K per pipeline stage */
  int32_t n_ktiles;        /* ceil(K_pad / bk) */
  int32_t tiles_per_split; /* K tiles one CTA walks */
  int32_t ctas;            /* grid_x * grid_y */
  int32_t smem_bytes;      /* dynamic shared memory per CTA */
  int64_t ws_floats;       /* FP32 partials the caller must supply; 0 if grid_y == 1 */
} chr_nf4_plan_t;

/* y[M,N] = bf16( sum_k bf16(LUT[code]*scale)[m,k] * x[k,n] ), FP32 accumulate.
 * x: bf16 [K, N] row-major (N fastest); y: bf16 [M, N]. N in [1, 32] for the
 * two plain entries, up to max_n (<= 64) for chr_nf4_gemm_ws_max.
 * Replaces gpu/include/chr_gpu.h:34 (chr_nf4_gemm), :72 (chr_nf4_gemm_ws),
 * :77 (chr_nf4_gemm_ws_max), :66 (chr_nf4_gemm_plan), :86 (chr_nf4_set_tuning);
 * kernels gpu/nf4/nf4_gemm.cu:1108-1130,1428-1450. */
int chr_nf4_gemm(const chr_nf4_dev_t *w, const void *x, void *y, int32_t N,
                 void *stream);
int chr_nf4_gemm_plan(const chr_nf4_dev_t *w, int32_t N, int32_t have_ws,
                      chr_nf4_plan_t *out);
int chr_nf4_gemm_ws(const chr_nf4_dev_t *w, const void *x, void *y, int32_t N,
                    float *ws, int64_t ws_floats, void *stream);
int chr_nf4_gemm_ws_max(const chr_nf4_dev_t *w, const void *x, void *y, int32_t N,
                        float *ws, int64_t ws_floats, void *stream, int32_t max_n);
/* path: 0 auto; split_k: 0 auto, >0 forced (clamped to the K tiles);
 * one_wave: SM count the split-K target is expressed in, 0 = this device. */
void chr_nf4_set_tuning(int32_t path, int32_t split_k, int32_t one_wave);

/* y[M] = bf16( sum_k (LUT[code]*scale)[m,k] * x[k] (+ add[m]) ), everything
 * FP32 until the single final rounding; weights are NOT rounded to bf16.
 * x bf16 [K]; y bf16 [M]; add optional bf16 [M], may alias y; rms_w optional
 * bf16 [K]: RMSNorm(x, rms_w, rms_eps) is applied to x first (rounded to bf16,
 * as a separate rms kernel would).
 * Replaces gpu/include/chr_gpu.h:94 ; kernel gpu/nf4/nf4_gemv.cu:291-324. */
int chr_nf4_gemv(const chr_nf4_dev_t *w, const void *x, void *y, void *stream,
                 const void *add, const void *rms_w, float rms_eps);

/* Three GEMVs sharing x in one launch, each with an optional bf16 bias [M].
 * q, k, v must share K and K_pad.
 * Replaces gpu/include/chr_gpu.h:101 ; kernel gpu/nf4/nf4_gemv.cu:326-390. */
int chr_nf4_gemv_qkv(const chr_nf4_dev_t *q, const chr_nf4_dev_t *k,
                     const chr_nf4_dev_t *v, const void *x, void *yq, void *yk,
                     void *yv, const void *bq, const void *bk, const void *bv,
                     void *stream, const void *rms_w, float rms_eps);

/* y[M] = bf16( silu(gate.x) * (up.x) ), silu(t) = t / (1 + expf(-t)).
 * Replaces gpu/include/chr_gpu.h:109 ; kernel gpu/nf4/nf4_gemv.cu:392-495. */
int chr_nf4_gemv_swiglu(const chr_nf4_dev_t *gate, const chr_nf4_dev_t *up,
                        const void *x, void *y, void *stream, const void *rms_w,
                        float rms_eps);

/* In-place rotate-half RoPE on q [n_q,hd] and k [n_kv,hd] (rounded to bf16),
 * then k and v are written to cache row *position. cos/sin bf16 [max_seq,hd];
 * position: device int64. A position outside [0,max_seq) writes nothing.
 * Replaces gpu/include/chr_gpu.h:116 ; kernel gpu/nf4/nf4_gemv.cu:497-537. */
int chr_nf4_rope_kv(void *q, void *k, const void *v, void *k_cache, void *v_cache,
                    const void *cos, const void *sin, const void *position,
                    int32_t n_q, int32_t n_kv, int32_t hd, int32_t max_seq,
                    void *stream);

/* GQA decode attention over cache rows t < *valid_len (device int32).
 * k, v: bf16 cache [max_seq, n_kv, hd]; q bf16 [n_q, hd]; out bf16 [n_q*hd];
 * ws: FP32 workspace of at least n_q*n_split*(hd+2) floats. With cos, sin and
 * position (device int64) q is rotated in FP32; with k_act/v_act as well, the
 * rotated current k and the current v are written to cache row *position and
 * the current token is attended with those unrounded FP32 values.
 * hd <= 256, hd % 8 == 0, n_split in [1, 64] (at most 32 splits are used, and fewer while splits x kv heads
 * x head chunks would exceed the SM count; the workspace is sized for n_split).
 * Cross-call state: the splits of a kv head are merged by the last CTA to arrive,
 * counted in a small array inside the library that every call leaves zeroed. Calls
 * that follow each other on one stream (or are otherwise ordered) are fine; two
 * attention launches that overlap on the device (different streams) share those
 * counters and must be serialised by the caller.
 * Replaces gpu/include/chr_gpu.h:123 ; kernels gpu/nf4/nf4_gemv.cu:599-727. */
int chr_nf4_attn(const void *q, const void *k, const void *v, void *out,
                 const void *valid_len, float *ws, int32_t n_q, int32_t n_kv,
                 int32_t hd, int32_t n_split, float scale, void *stream,
                 const void *k_act, const void *v_act, const void *cos,
                 const void *sin, const void *position, int32_t max_seq);

/* chr_nf4_attn for `batch` independent sequences in one launch (batched decode):
 * q [batch, n_q, hd], k_act / v_act [batch, n_kv, hd], k / v caches
 * [batch, max_seq, n_kv, hd], out [batch, n_q*hd], valid_len int32 [batch],
 * position int64 [batch], ws batch * n_q*min(n_split,32)*(hd+2) floats; cos / sin
 * are shared. batch * n_kv * ceil(n_rep / 8) must not exceed 1024 (-3). Same
 * arithmetic per sequence as chr_nf4_attn. No counterpart in the reference, whose
 * decode is one sequence (gpu/nf4/nf4_gemv.cu:599-727). */
int chr_nf4_attn_batch(const void *q, const void *k, const void *v, void *out,
                       const void *valid_len, float *ws, int32_t batch, int32_t n_q,
                       int32_t n_kv, int32_t hd, int32_t n_split, float scale, void *stream,
                       const void *k_act, const void *v_act, const void *cos,
                       const void *sin, const void *position, int32_t max_seq);

/* y[i] = bf16( w[i] * x[i] * rsqrt(mean(x^2) + eps) ); x, w, y bf16 [n].
 * Replaces gpu/include/chr_gpu.h:133 ; kernel gpu/nf4/nf4_gemv.cu:729-751. */
int chr_nf4_rms(const void *x, const void *w, void *y, int32_t n, float eps,
                void *stream);

/* ------------------------------------------------------------------------ */
/* Additive entries (no counterpart in the reference's header)               */
/* ------------------------------------------------------------------------ */

/* Library identification: "chr_nf4 sm_100a <build tag>". */
const char *chr_nf4_version(void);

/* chr_nf4_gemv with the FP32 sum stored unrounded (y: device float [M]): the
 * partial result of a row-split (tensor-parallel) linear, to be summed across
 * ranks before the single bf16 rounding. add: optional bf16 [M] (e.g. a bias). */
int chr_nf4_gemv_f32(const chr_nf4_dev_t *w, const void *x, float *y, void *stream,
                     const void *add, const void *rms_w, float rms_eps);

/* GEMV for N = 1..8 activation rows on CUDA cores: y_rows[n, :] = bf16( dequant(W) .
 * x_rows[n, :] (+ bias) (+ add_rows[n, :]) ) with the numerics of chr_nf4_gemv (FP32
 * weights LUT*scale, never rounded to bf16; FP32 accumulation; one rounding). A pass
 * over the weights serves up to four rows (every packed weight is read from HBM once
 * and looked up once for all of them); five to eight rows take two passes. It is what
 * batched decode wants where the tensor-core GEMM's bf16 weights are not.
 * x_rows bf16 [N, K]; y_rows bf16 [N, M]; add_rows optional bf16 [N, M] (may alias
 * y_rows); bias optional bf16 [M]. K beyond 11264 is cut into slices whose FP32
 * partials go to ws ([slices, min(N, 4), M], reused by the second pass);
 * chr_nf4_gemv_n_ws says how many floats that takes (0 when one slice covers K); a
 * missing or small ws -> -7; N outside 1..8 -> -2.
 * No counterpart in the reference (its GEMV is N = 1, gpu/nf4/nf4_gemv.cu:291-324). */
int64_t chr_nf4_gemv_n_ws(const chr_nf4_dev_t *w, int32_t N);
int chr_nf4_gemv_n(const chr_nf4_dev_t *w, const void *x_rows, void *y_rows, int32_t N,
                   const void *add_rows, const void *bias, float *ws, int64_t ws_floats,
                   void *stream);

/* Work split the GEMV family uses for a matrix of n_rows x K_pad (swiglu != 0: the
 * gate/up pair): out = {R rows per warp and tile, C 1024-wide chunks per warp, S K
 * slices, G row groups per CTA, tiles, CTAs}. Host-only (no launch); -3 when K_pad is beyond
 * what the kernels cover. Ranks of a tensor-parallel group that pass the same
 * arguments get the same split, which chr_nf4_gemv_allreduce relies on. */
int chr_nf4_gemv_shape(int32_t n_rows, int32_t K_pad, int32_t swiglu, int32_t out[6]);

/* Row-split linear of a tensor-parallel shard with the exchange fused in: ONE
 * launch per rank computes this rank's FP32 partial W_shard . x_shard, pushes every
 * row into every peer's receive buffer over NVLink as one 8-byte word (value, call
 * epoch) with plain peer stores, polls (bounded) its own buffer for the peers' words of
 * the same rows, sums the partials in rank order, adds the residual and rounds once:
 *   y[m] = bf16( f32(y[m]) + sum_r partial_r[m] )      (y: bf16 [M], in place)
 * Every rank ends with the same y. The same CTA owns the same rows on every rank
 * (same matrix shape, same GPU model). No fence and no separate flag is on the path:
 * the word carries its own arrival mark.
 * Buffers (all device memory, mapped into every rank's address space, e.g.
 * symmetric memory or CUDA IPC; zeroed once before the first call):
 *   recv[p]  rank p's receive buffer: 2 * world * capacity 8-byte words (two halves
 *            that calls alternate between x one slot of `capacity` rows per source
 *            rank); M > capacity -> -7;
 *   flags[p] rank p's flag words: world * CHR_NF4_AR_MAX_CTAS uint32 (used by
 *            chr_nf4_pick_commit_tp, not by this entry);
 *   epoch    this rank's own uint32[2] {calls completed, exit ticket};
 *   status   this rank's own int32, set to 1 when a wait ran out of polls
 *            (2^22 unless chr_nf4_set_peer_polls changed it; the sum then leaves
 *            the missing partials out, and later calls stop waiting until the host
 *            clears the word).
 * All ranks must issue the same sequence of calls on these buffers and tile the
 * rows alike: when the ranks' K shares differ, each passes the largest K_pad of
 * the layer in shape_k_pad. Capturable
 * (the epoch lives in device memory). No counterpart in the reference. */
#define CHR_NF4_AR_MAX_RANKS 8
#define CHR_NF4_AR_MAX_CTAS 256

typedef struct {
  int32_t rank, world;
  int32_t shape_k_pad; /* 0, or the largest K_pad any rank holds for this layer (uneven shares) */
  int32_t capacity;    /* rows one source rank's slot of a receive buffer holds */
  void *recv[CHR_NF4_AR_MAX_RANKS];
  void *flags[CHR_NF4_AR_MAX_RANKS];
  void *epoch;
  void *status;
} chr_nf4_peers_t;

int chr_nf4_gemv_allreduce(const chr_nf4_dev_t *w, const void *x, void *y,
                           const chr_nf4_peers_t *peers, const void *add, void *stream);

/* Poll budget of the peer-flag wait above (process-wide; 0 restores 2^22). A small
 * budget lets a test see the wait run out without a peer having to fail. */
void chr_nf4_set_peer_polls(uint32_t polls);

/* Reads and clears the GEMV family's device status word (synchronises the device):
 * 0 = fine; 3001 = a kernel found its shared-memory window smaller than its layout
 * and did not run; 3002 = a bounded wait for a weight tile's bulk copy ran out and
 * the kernel returned early. In both cases the launch's output is undefined. */
int chr_nf4_gemv_status(void);

/* Wide GEMM on activation rows: y_rows[N, M] = bf16( x_rows[N, K] . dequant(W)^T ),
 * the layout activations already have ([tokens, features], K contiguous), so no
 * transposes on either side and any N >= 1 in one call (tiled 16..256 columns per
 * CTA). Same tcgen05 pipeline and numerics as chr_nf4_gemm; the activation tile is
 * loaded by TMA, which needs K % 8 == 0 (-3 otherwise) and x_rows 16-byte aligned.
 * ws: optional FP32 split-K workspace of chr_nf4_gemm_rows_ws(w, N) floats (0 = the
 * shape fills the GPU without split-K); NULL pins split-K to 1; too small -> -7.
 * Replaces the transpose + chunk loop around chr_nf4_gemm in
 * gpu/decodev2/linear.py:101-136 and gpu/host/linear.py:31-81. */
int64_t chr_nf4_gemm_rows_ws(const chr_nf4_dev_t *w, int32_t N);
int chr_nf4_gemm_rows(const chr_nf4_dev_t *w, const void *x_rows, void *y_rows, int32_t N,
                      float *ws, int64_t ws_floats, void *stream);

/* chr_nf4_gemm_rows with the bias and a residual folded into the epilogue:
 *   y_rows[n, m] = bf16( sum_k ... + f32(bias[m]) + f32(add_rows[n, m]) )
 * one rounding instead of one per torch op (the reference adds bias and residual as
 * bf16 tensor ops after the GEMM, gpu/decodev2/linear.py:131-133,
 * gpu/decodev2/prefill.py:118-131). bias: optional bf16 [M]; add_rows: optional bf16
 * [N, M], may alias y_rows. With split-K the reduction kernel does the adding. */
int chr_nf4_gemm_rows_add(const chr_nf4_dev_t *w, const void *x_rows, void *y_rows, int32_t N,
                          const void *bias, const void *add_rows, float *ws, int64_t ws_floats,
                          void *stream);

/* Programmatic dependent launch for the decode-chain kernels (GEMV family,
 * attention, embedding rows, pick): on (default, or CHR_NF4_PDL=1) lets a kernel's
 * prologue overlap the previous kernel's tail, inside CUDA graphs as well; 0
 * restores plain stream order. Results are identical either way. */
void chr_nf4_set_pdl(int32_t on);

/* Reads and clears the tensor-core GEMM's device status word (synchronises the
 * device): 0 = every bounded pipeline wait completed; 1..4 = the TMA producer /
 * MMA issuer / dequant warps / epilogue gave up on a wait and the affected
 * launch's output is undefined. */
int chr_nf4_gemm_status(void);

/* Rows ids[0..n) of an NF4 table decoded to bf16( f32(LUT)*f32(scale) ),
 * out bf16 [n, K]. ids: device int64. An id outside [0, M) yields a zero row
 * and sets *status (device int32, optional) to 1. When position and valid_len
 * are both non-null (device int64 / int32), *valid_len = *position + 1 is
 * stored as well, which is what the greedy step needs before attention.
 * Replaces the torch-op row decode gpu/host/embedding.py:74-107 (called from
 * gpu/decodev2/embed.py:39-50). */
int chr_nf4_embed_rows(const chr_nf4_dev_t *w, const void *ids, int32_t n,
                       void *out, void *status, const void *position,
                       void *valid_len, void *stream);

/* Greedy pick and commit in one launch: next = argmax(logits[0..n)) (lowest
 * index on ties, NaN counts as the maximum), then *next_token = next,
 * *token = next, *position += 1, *finished |= (next == eos). logits bf16;
 * next_token/token/position device int64; finished device uint8; token,
 * position and finished may be NULL (pick only). scratch: 16 zero-initialised
 * device bytes owned by the caller; the kernel leaves them zero again.
 * Replaces the torch ops gpu/decodev2/step.py:182 and state.py:98-103. */
int chr_nf4_pick_commit(const void *logits, int32_t n, void *next_token,
                        void *token, void *position, void *finished,
                        int64_t eos, void *scratch, void *stream);

/* chr_nf4_pick_commit for B sequences in one launch: logits bf16 [B, n] (rows
 * row_stride elements apart), next_token / token / position int64 [B], finished
 * uint8 [B] (token, position, finished optional), scratch B x 16 bytes (8-byte
 * aligned, zeroed once; every launch leaves it zeroed). Same pick per sequence as the
 * one-sequence entry (lowest index on ties, NaN above everything). Batched decode is
 * not in the reference (gpu/decodev2/step.py:182 picks one sequence). */
int chr_nf4_pick_commit_batch(const void *logits, int64_t row_stride, int32_t n, int32_t batch,
                              void *next_token, void *token, void *position, void *finished,
                              int64_t eos, void *scratch, void *stream);

/* chr_nf4_pick_commit when the logits are split over a tensor-parallel group: this rank
 * holds logits_local[0..n_local) = vocabulary ids index_offset..index_offset+n_local-1.
 * Each rank picks its local best, exchanges that one (value, id) pair with every peer
 * over the mapped buffers of `peers` (plain peer stores + a flag per peer, bounded wait,
 * sticky status word, as chr_nf4_gemv_allreduce) and all ranks commit the same global
 * argmax: two scalars per rank cross NVLink instead of the logits. The peers struct
 * must be a set of its own (its epoch advances once per call); capacity >= 2.
 * No counterpart in the reference (single GPU). */
int chr_nf4_pick_commit_tp(const void *logits_local, int32_t n_local, int32_t index_offset,
                           const chr_nf4_peers_t *peers, void *next_token, void *token,
                           void *position, void *finished, int64_t eos, void *scratch,
                           void *stream);

/* chr_nf4_attn without the workspace argument, for callers that have no way to
 * allocate device memory (a pointer-forwarding binding, a plugin without access
 * to the host's memory pool, code under a no-allocation rule). No counterpart in
 * the reference. The split partials go to a 1 MiB array built into the library
 * (resident on every GPU that loads it); the call returns -7 when
 * n_q * min(n_split, 32) * (hd + 2) exceeds 262144 floats. It calls no
 * allocation routine. The first call on a device looks the array's address up
 * (one host-side runtime query) and should therefore come before any stream
 * capture on that device; the device that owns `stream` must be the current one. All calls share the array: nothing in it has to start
 * at zero, but two calls that overlap on the GPU (different streams, or another
 * process thread) race on it and must be serialised by the caller. */
int chr_nf4_attn_noalloc(const void *q, const void *k, const void *v, void *out,
                         const void *valid_len, int32_t n_q, int32_t n_kv, int32_t hd,
                         int32_t n_split, float scale, void *stream, const void *k_act,
                         const void *v_act, const void *cos, const void *sin,
                         const void *position, int32_t max_seq);

/* Host-side NF4 codec, bit-exact with the reference's encoder/decoder
 * (internal/nf4/nf4.go:46-121,129-185; gpu/tests/nf4_oracle.py:119-187).
 * w: host float32 [M, K]; packed: host [M, K_pad/2]; scale: host binary16 bits
 * [M, K_pad/64]. threads <= 0 uses every core. Returns 0, -1 (null), -3 (dims)
 * or -8 (non-finite input). A group scale outside binary16's finite positive
 * range is clamped as the Go writer does. */
int chr_nf4_encode_f32(const float *w, int32_t M, int32_t K, uint8_t *packed,
                       uint16_t *scale, int32_t threads);
int chr_nf4_decode_f32(const uint8_t *packed, const uint16_t *scale, int32_t M,
                       int32_t K, float *w, int32_t threads);

/* The same encoder on the device, one warp per group: w device float32 [M, K],
 * packed / scale device blobs of the shapes above, status optional device int32
 * set to 1 when a non-finite weight is met. Bit-identical to the host encoder. */
int chr_nf4_encode_dev(const float *w, int32_t M, int32_t K, uint8_t *packed,
                       uint16_t *scale, int32_t *status, void *stream);

/* ---- Row-wise helpers of the chunked prefill -------------------------------
 * The elementwise work between a chunk's GEMMs, which the reference issues as
 * torch ops in the cache dtype (gpu/decodev2/prefill.py:58-141); one launch each.
 * No counterpart in the reference's C ABI. */

/* y[n, :] = bf16( w * x[n, :] * rsqrt(mean(x[n, :]^2) + eps) ) for N rows of K bf16
 * values; x rows x_stride elements apart (a multiple of 8), y contiguous. The same
 * summation order as chr_nf4_rms and the GEMVs' fused RMSNorm. */
int chr_nf4_rms_rows(const void *x, int64_t x_stride, const void *w, void *y, int32_t N,
                     int32_t K, float eps, void *stream);

/* Causal GQA attention of one prefill chunk (additive entry; the reference runs
 * torch's scaled_dot_product_attention with a boolean mask per chunk,
 * gpu/decodev2/prefill.py:50-92). Query row i (0 <= i < n, position start + i) attends
 * cache rows t <= start + i:
 *   out[i, h, :] = softmax_t( scale * q[i, h, :] . k_cache[t, h / n_rep, :] ) . v_cache[t, ...]
 * q: bf16 [n, n_q, hd], rows q_stride elements apart (even, >= n_q*hd), already
 * rotated; k_cache, v_cache: bf16 [max_seq, n_kv, hd] holding rows 0 .. start+n-1
 * (the chunk's own rows included); out: bf16 [n, n_q*hd] contiguous. FP32 scores,
 * running softmax and accumulation; the probabilities are rounded to bf16 for the
 * value product. hd in {16, 32, 64, 128}; start + n <= max_seq. No mask tensor, no
 * workspace. Capturable. Returns 0 or a negative code (-1 null, -3 dims,
 * -5 alignment: caches 16 bytes, q / out 4 bytes, -6 launch). */
int chr_nf4_attn_prefill(const void *q, int64_t q_stride, const void *k_cache,
                         const void *v_cache, void *out, int32_t n, int32_t start,
                         int32_t n_q, int32_t n_kv, int32_t hd, int32_t max_seq, float scale,
                         void *stream);

/* RoPE for N consecutive positions start..start+N-1 and the cache write of the
 * chunk: q [N, n_q, hd] (rows q_stride apart) is rotated into q_out (contiguous),
 * k is rotated into k_cache rows, v copied into v_cache rows (caches bf16
 * [max_seq, n_kv, hd]). bf16 arithmetic with a rounding after each product and
 * after the sum, as torch's tensor math in bf16 does. */
int chr_nf4_rope_kv_rows(const void *q, int64_t q_stride, const void *k, int64_t k_stride,
                         const void *v, int64_t v_stride, void *q_out, void *k_cache,
                         void *v_cache, const void *cos, const void *sin, int32_t start,
                         int32_t N, int32_t n_q, int32_t n_kv, int32_t hd, int32_t max_seq,
                         void *stream);

/* out[n, i] = bf16( bf16(silu(g)) * u ) with g = gate_up[n, i], u = gate_up[n, I + i]:
 * the activation on the output of the stacked gate/up GEMM (bf16 [N, 2*I]). */
int chr_nf4_silu_mul(const void *gate_up, void *out, int32_t N, int32_t I, void *stream);

#ifdef __cplusplus
}
#endif
