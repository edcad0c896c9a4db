/*
 * triteia_b200 — C ABI of the B200 (sm_100a) indexed low-precision delta matmul library.
 *
 * Every entry point takes raw DEVICE pointers, plain integers and a CUDA stream handle
 * (cudaStream_t passed as void*), returns an int status (0 = ok) and allocates nothing:
 * outputs, workspaces and scratch buffers are owned by the caller, exactly as in the
 * reference, whose launchers these functions replace.  Citations name files of the
 * reference project (eth-easl/triteia).
 *
 * Tensor conventions (K = input features, N = output features, T = tokens, D = deltas):
 *   x / A      fp16 [T, K] row-major
 *   qweight    int32 [K/32, 2N]        (stacked: [D, K/32, 2N])
 *   meta       int16 [N, K/16]         (stacked: [D, N, K/16])
 *   scales     fp16 [G, N], G = 1 (per output channel) or K/128 (per group of 128 K),
 *              stacked [D, G, N]; `groupsize` below is -1 or 128 (dense-K units)
 *   y / C      fp16 [T, N] row-major
 */
#ifndef TRITEIA_B200_H_
#define TRITEIA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  1 and 2 keep the reference's values (csrc/ops/marlin_nm.cu:39-40). */
#define TRB_OK 0
#define TRB_ERR_PROB_SHAPE 1   /* problem shape not supported (N % 128, K % 128, group size) */
#define TRB_ERR_KERN_SHAPE 2   /* no kernel instantiation for the request */
#define TRB_ERR_BAD_ARG 3      /* null pointer, misaligned pointer, negative size */
#define TRB_ERR_CUDA 4         /* a CUDA runtime / driver call failed */
#define TRB_ERR_TIMEOUT 5      /* a bounded device-side wait expired (see trb_device_status) */
#define TRB_ERR_SCRATCH 6      /* caller-provided scratch buffer too small */

/* dtype tags for the LoRA entry points */
#define TRB_F16 0
#define TRB_BF16 1

int trb_version(void);
const char* trb_status_string(int status);

/* Reads and clears the device-side error word of device `dev` (synchronises `dev`).
 * 0 = no kernel reported a problem since the last call; TRB_ERR_TIMEOUT = a bounded wait
 * inside a kernel expired and that launch's output is invalid.
 * No counterpart in the reference (its device code spins without bound,
 * csrc/ops/common/mem.h:112-124). */
int trb_device_status(int dev, int* status_out);

/* Self-test of the bounded device-side waits: launches one CTA that waits, for at most max_polls
 * polls (1 .. 1 000 000), on a barrier nothing ever signals.  The wait expires, the kernel stores 1
 * into *gave_up_flag (device int, may be NULL), records TRB_ERR_TIMEOUT in the device error word and
 * ends normally: after it trb_device_status reports TRB_ERR_TIMEOUT once, then 0.  No counterpart in
 * the reference (its waits have no limit, csrc/ops/common/mem.h:112-124). */
int trb_selftest_timeout(int max_polls, void* gave_up_flag, int dev, void* stream);

/* C[T,N] = A[T,K] @ dequant(B, meta, s).  Overwrites C.
 * Replaces marlin::marlin_cuda_2_4 (csrc/ops/marlin_nm.cu:42-119), same argument order:
 * prob_m = N (output features), prob_n = T (tokens), prob_k = K.  `groupsize` is in dense-K
 * units here (-1 or 128).  `workspace`, thread_k, thread_m, sms (limits the CTA count when
 * > 0) and max_par are accepted for call compatibility; workspace is not touched. */
int trb_mul_2_4(const void* A, const void* B, const void* meta, void* C, const void* s,
                int prob_m, int prob_n, int prob_k, void* workspace, int groupsize, int dev,
                void* stream, int thread_k, int thread_m, int sms, int max_par);

/* Selective batched matmul over R segments: for r < prob_r,
 *   C[starts[r] : starts[r]+counts[r]] = A[same rows] @ dequant(B[indices[r]], ...).
 * Rows of C outside every segment are not written.  indices/starts/counts: int32 [R] on the
 * device.  Replaces triteia::triteia_cuda_sbmm_2_4 (csrc/ops/triteia_nm_sbmm.cu:809-847),
 * same argument order (prob_m = N, prob_n = T, prob_k = K, prob_r = R).  Unlike the
 * reference, per-group scales are honoured and all segments run concurrently in ONE launch. */
int trb_sbmm_2_4(const void* A, const void* B, const void* meta, void* C, const void* s,
                 const void* indices, const void* starts, const void* counts, int prob_m,
                 int prob_n, int prob_k, int prob_r, void* workspace, int groupsize, int dev,
                 void* stream, int thread_k, int thread_m, int sms, int max_par);

/* One weight per request: C[b, 0, :] = A[b, 0, :] @ dequant(B[b], meta[b], s[b]), b < prob_n.
 * Replaces triteia::triteia_cuda_bmm_2_4 (csrc/ops/triteia_nm_bmm.cu:760-834). */
int trb_bmm_2_4(const void* A, const void* B, const void* meta, void* C, const void* s,
                int prob_m, int prob_n, int prob_k, void* workspace, int groupsize, int dev,
                void* stream, int thread_k, int thread_m, int sms, int max_par);

/* Token router: groups T tokens by delta id (stable, id -1 first) and builds the tile work
 * list that the grouped kernel consumes.  Replaces the torch prologue of
 * triteia/python/ops/matmul/sbmm.py:94-123 (unique_consecutive + cumsum + 3 host syncs) with
 * one launch and no host synchronisation; indices may be in ANY order.
 *   indices   int32 [T]; id = indices[t] - index_offset selects the delta, ids outside
 *             [0, num_deltas) (this includes -1) mean "no delta for this token"
 *   perm      int32 [T]   out: token positions in sorted order
 *   seg_delta/seg_start/seg_count int32 [min(T, num_deltas)] out: one entry per distinct
 *             delta id >= 0 in increasing id order; start/count index the SORTED order
 *   tile_delta/tile_start/tile_count int32 [trb_route_max_tiles(T, num_deltas, tile_tokens)]
 *             out: segments cut into tiles of at most tile_tokens tokens
 *   counters  int32 [4] out: {R, number of tiles, number of tokens with id -1,
 *             number of raw indices < -1 or >= index_offset + num_deltas}
 * Any of perm / seg_* / tile_* may be NULL to skip that output.  T <= 65536,
 * num_deltas <= 8191. */
int trb_route(const void* indices, int num_tokens, int num_deltas, int tile_tokens,
              int index_offset, void* perm, void* seg_delta, void* seg_start, void* seg_count, void* tile_delta,
              void* tile_start, void* tile_count, void* counters, int dev, void* stream);
int trb_route_max_tiles(int num_tokens, int num_deltas, int tile_tokens);

/* trb_sbmm_2_4 with working memory for the small-tile kernel's tail K split: when the last round
 * of work items covers at most half of the SMs, its items are cut along K and the pieces are summed
 * in a fixed order by whichever piece finishes last.  `ksplit`: trb_sbmm_ksplit_bytes() bytes,
 * 256-byte aligned, first 512 bytes zero on entry (zero again when the launch has finished);
 * nullptr = plain trb_sbmm_2_4.  No counterpart in the reference (its K split goes through the
 * lock workspace, marlin_cuda_kernel_nm.cu). */
size_t trb_sbmm_ksplit_bytes(void);
int trb_sbmm_2_4_ksplit(const void* A, const void* B, const void* meta, void* C, const void* s,
                        const void* indices, const void* starts, const void* counts, int prob_m,
                        int prob_n, int prob_k, int prob_r, int groupsize, int dev, void* stream,
                        void* ksplit, size_t ksplit_bytes);

/* Fused indexed delta matmul: y[t] (+)= x[t] @ dequant(delta[indices[t] - index_offset]) for
 * indices[t] - index_offset in [0, num_deltas); other tokens count as "index -1".
 * Router + row gather + grouped kernel on `stream`, no host synchronisation; indices in any
 * order.  accumulate != 0: y[t] += ...  (rows with index -1 untouched); accumulate == 0:
 * rows with index >= 0 are overwritten, rows with index -1 are set to zero.
 * Stands for the body of sbmm_4bit_2_4_native (triteia/python/ops/matmul/sbmm.py:89-142)
 * after its base GEMM.  `scratch` should hold trb_sbmm_indexed_scratch_bytes(T, K, D) bytes
 * (mirrors sgmv_tmp_size, csrc/ops/sgmv.cuh:48-52) and must hold at least
 * trb_sbmm_indexed_scratch_min_bytes(T, K, D); the difference (1.2 MB) is the room for the
 * partial tiles of the small-tile kernel's tail K split, which is left out when it is missing. */
size_t trb_sbmm_indexed_scratch_bytes(int num_tokens, int prob_k, int num_deltas);
size_t trb_sbmm_indexed_scratch_min_bytes(int num_tokens, int prob_k, int num_deltas);
int trb_sbmm_indexed(const void* x, const void* qweights, const void* metas, const void* scales,
                     const void* indices, void* y, int num_tokens, int prob_m, int prob_k,
                     int num_deltas, int index_offset, int groupsize, int accumulate,
                     void* scratch, size_t scratch_bytes, int dev, void* stream);

/* trb_sbmm_indexed in two calls with the same arguments and the same scratch: phase 1 = router +
 * row gather (with accumulate != 0 they write nothing but the scratch, so they may run on another
 * stream beside the kernel that produces y, e.g. the base product of ldmm), phase 2 = the grouped
 * kernels, phase 3 = both (= trb_sbmm_indexed).  The caller orders phase 2 after phase 1. */
int trb_sbmm_indexed_phase(const void* x, const void* qweights, const void* metas, const void* scales,
                           const void* indices, void* y, int num_tokens, int prob_m, int prob_k,
                           int num_deltas, int index_offset, int groupsize, int accumulate,
                           void* scratch, size_t scratch_bytes, int phase, int dev, void* stream);

/* trb_sbmm_indexed without a scratch argument, for hosts that cannot allocate device memory for
 * the library (a server whose arena owns all of HBM and offers foreign code no allocator, a plugin
 * contract that bans cudaMalloc after start-up because it stalls the whole device).  The working
 * memory is a fixed array inside the library image: trb_sbmm_indexed_static_capacity() bytes
 * (4 MiB + 64 KiB), held by every GPU that uses the library until the process exits.  A request
 * whose trb_sbmm_indexed_scratch_min_bytes() exceeds the capacity returns TRB_ERR_SCRATCH and launches
 * nothing (fits e.g. 256 tokens x K 8192, or 512 tokens x K 4096).  Calls no allocator of any kind.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current); make that first call before any stream capture begins.  All calls on a device
 * share the one array and it keeps the previous call's contents: nothing in it needs clearing
 * between calls, but two calls that overlap on the GPU (different streams, no ordering) race.
 * This entry point has no counterpart in the reference. */
size_t trb_sbmm_indexed_static_capacity(void);
int trb_sbmm_indexed_static(const void* x, const void* qweights, const void* metas,
                            const void* scales, const void* indices, void* y, int num_tokens,
                            int prob_m, int prob_k, int num_deltas, int index_offset, int groupsize,
                            int accumulate, int dev, void* stream);

/* Multi-GPU form: deltas sharded by id over `world` ranks (owner = id % world, local id =
 * id / world).  Tokens travel through fixed-capacity exchange buffers of `world` chunks of
 * num_tokens + 1 rows (trb_shard_buffer_rows rows in all): outbound rows of K halves with the rows'
 * local ids and the row count in each chunk's last row, return rows of N halves in the same slots.
 * Between the calls the host runs an all-to-all with equal splits (NCCL); nothing here needs a count
 * on the host.  The reference has no distributed layer: no counterpart.
 *   trb_shard_dispatch  plan the slots (slot_of int32 [T] out, plan int32 [8 + world] scratch) and
 *                       pack this rank's rows and ids into send_buf
 *   trb_shard_compute   on the owner: router + gather + grouped kernel over the received buffer
 *                       (cap = the senders' num_tokens); scratch as trb_sbmm_indexed for
 *                       world * (cap + 1) tokens
 *   trb_shard_combine   y[t] (+)= returned row of token t; tokens without a delta are zeroed unless
 *                       accumulate
 * Peer form (no collective at all): peer_recv_ptrs / peer_out_ptrs are device arrays of `world`
 * pointers to every rank's receive buffer / output tensor [num_tokens, N] (peer-mapped memory, e.g.
 * CUDA symmetric memory).  The pack kernel stores rows straight into the owner's receive buffer over
 * NVLink (chunk index = my_rank) and clears the rows of y_zero (this rank's output tensor) whose
 * token has no delta; the grouped kernel's epilogue stores every result row straight into the
 * source rank's output tensor at the token's own row.  The host only places a cross-GPU barrier
 * after each of the two calls; trb_shard_combine is not used.  Pass NULL for the plain form. */
size_t trb_shard_buffer_rows(int num_tokens, int world);
int trb_shard_dispatch(const void* x, const void* indices, int num_tokens, int prob_k, int world,
                       void* send_buf, const void* peer_recv_ptrs, int my_rank, void* y_zero,
                       int prob_m, void* slot_of, void* plan, int dev, void* stream);
int trb_shard_compute(const void* recv_buf, const void* qweights, const void* metas,
                      const void* scales, void* y_work, int world, int cap, int prob_m, int prob_k,
                      int num_local_deltas, int groupsize, const void* peer_out_ptrs, int my_rank,
                      void* scratch, size_t scratch_bytes, int dev, void* stream);
int trb_shard_combine(const void* back_buf, const void* slot_of, void* y, int num_tokens, int prob_m,
                      int world, int accumulate, int dev, void* stream);

/* Dense fp16 weight [K, N] from a packed delta (W = fp16(level) * fp16(scale), rounded once).
 * The on-GPU statement of the format; bit-exact against the CPU decoder.  No counterpart
 * kernel in the reference (its decoder is torch code,
 * triteia/python/ops/utils/sparsity.py:297-394). */
int trb_unpack_2_4(const void* B, const void* meta, const void* s, void* w_out, int prob_m,
                   int prob_k, int groupsize, int dev, void* stream);

/* The packer as a kernel: fp16 weight [K, N] (K = prob_k input features, N = prob_m output features;
 * the two largest magnitudes of every four K positions are kept) and logical scales fp16 [G, N]
 * (G = 1 or K / 128) -> qweight int32 [K/32, 2N], meta int16 [N, K/16] (physical order), stored
 * scales fp16 [G, N].  Same result as the reference's host packer
 * (triteia/python/nn/linear.py:79-141) for weights that are already 2:4 sparse; K % 128 == 0,
 * N % 256 == 0 as there. */
int trb_pack_2_4(const void* weight_kn, const void* scales_logical, void* qweight, void* meta,
                 void* scales_stored, int prob_k, int prob_m, int groupsize, int dev, void* stream);

/* Element-wise neighbours of the linears, as the reference's extension offers them.
 * trb_gelu_quick: out = x * sigmoid(1.702 x) over numel elements (numel % 8 == 0, 16-byte aligned);
 *   replaces vllm::gelu_quick (csrc/ops/activations.cu:203-207).
 * trb_silu_and_mul: out[t, :d] = silu(in[t, :d]) * in[t, d:2d] (d % 8 == 0); replaces silu_and_mul
 *   (activations.cu:68-72).
 * trb_rotary_embedding: in-place GPT-NeoX (is_neox) or GPT-J rotation of the first rot_dim elements
 *   of every head; positions int64 [T], cos_sin_cache [max_position, rot_dim], strides in elements,
 *   key may be NULL; cache_offsets int64 [T] or NULL (the batched form).  Replaces
 *   rotary_embedding / batched_rotary_embedding (csrc/ops/pos_encoding_kernels.cu:118-213).
 * dtype: TRB_F16 or TRB_BF16. */
int trb_gelu_quick(void* out, const void* in, long long numel, int dtype, int dev, void* stream);
int trb_silu_and_mul(void* out, const void* in, int num_tokens, int d, int dtype, int dev, void* stream);
int trb_rotary_embedding(const void* positions, void* query, void* key, const void* cos_sin_cache,
                         const void* cache_offsets, int num_tokens, int rot_dim, long long query_stride,
                         long long key_stride, int num_heads, int num_kv_heads, int head_size,
                         int is_neox, int dtype, int dev, void* stream);

/* sums[r] = (accumulate ? sums[r] : 0) + sum over n of y[r, n]: fp32 per-row checksum of an fp16
 * matrix [rows, prob_m] (prob_m % 8 == 0, y 16-byte aligned), fixed summation order.  Used by the
 * sharded linear-stack scenario (a full Llama-2-7B-shaped stack of independent delta linears) to return
 * one number per token and linear instead of every output row.  No counterpart in the reference. */
int trb_row_checksum(const void* y, void* sums, int rows, int prob_m, int accumulate, int dev,
                     void* stream);

/* One pass of a stack of n_linears independent delta linears over one routed batch, issued from C
 * with no host read in between.  ids[r] (int32, device) selects the delta of row r in EVERY linear
 * (ids outside [0, num_deltas): no delta, outputs count as zero), so rows are routed once: one router
 * launch, one row gather per input width, then per linear the tcgen05 launch (segments of more than
 * 32 rows; only when rows > 128), the mma.sp launch (8-row tiles, tail K split) and the fold of the
 * output into the per-row checksum (trb_row_checksum semantics).  Host arrays of device pointers /
 * ints: x_of_width[w] [rows, width[w]] fp16 in the caller's row order, xs_of_width[w] scratch of the
 * same size, k[i] (one of width[]) and n[i] the shape of linear i, y_of[i] [rows, n[i]] fp16 scratch
 * (buffers of one n may be shared).  y_last [rows, n[n_linears-1]]: output of the last linear in the
 * caller's row order; checksum [rows] fp32, caller's row order, ADDED to.  scratch:
 * trb_stack_scratch_bytes(rows, num_deltas) bytes, 256-byte aligned, no initial contents needed.
 * No counterpart in the reference. */
size_t trb_stack_scratch_bytes(int rows, int num_deltas);
int trb_stack_pass(int n_linears, const void* const* q, const void* const* meta,
                   const void* const* s, const int* k, const int* n, int n_widths, const int* width,
                   const void* const* x_of_width, void* const* xs_of_width, void* const* y_of,
                   void* y_last, const void* ids, int rows, int num_deltas, void* checksum,
                   int groupsize, void* scratch, size_t scratch_bytes, int dev, void* stream);

/* BGMV: Y[b, :] += scale * W[indices[b], layer_idx] @ X[b, :], W [M, L, h_out, h_in]
 * contiguous, indices int64 [B].  Replaces bgmv_kernel<feat_in, feat_out, T>
 * (csrc/ops/bgmv_config.h:3-7, csrc/ops/bgmv_impl.cuh:186-207); any h_in, h_out that are
 * multiples of 8 and < 65536 are accepted, and the launch goes to `stream` (the reference
 * always uses the legacy default stream, bgmv_impl.cuh:198-205). */
int trb_bgmv(void* Y, const void* X, const void* W, const void* indices, int batch, int h_in,
             int h_out, int num_layers, int layer_idx, float scale, int dtype, int dev,
             void* stream);

/* Fused LoRA for decode: y[b] += scale * (x[b] @ A[idx]) @ B[idx] in ONE launch, the rank-r
 * intermediate kept on chip.  wa_t [M, L, r, h1], wb_t [M, L, h2, r] (the layouts
 * add_lora_bgmv takes, triteia/python/capi/punica.py:34-68); indices int64 [B], a negative
 * index skips the row.  r <= 64. */
int trb_lora_bgmv_fused(void* y, const void* x, const void* wa_t, const void* wb_t,
                        const void* indices, int batch, int h1, int h2, int rank, int num_layers,
                        int layer_idx, float scale, int dtype, int dev, void* stream);

/* Indexed LoRA on the layouts the Python ops take: y[b] += scale * (x[b] @ A[id]) @ B[id] with
 * A [M, h1, r], B [M, r, h2], id = indices[b] (int32, or int64 when index_is_64bit); ids outside
 * [0, num_adapters) skip the row, so one index vector can address adapters and deltas.  Stands
 * for lora_bgmv / the LoRA branch of ldmm (triteia/python/ops/matmul/lora.py:22-48,
 * triteia/python/ops/matmul/ldmm.py:86-107) without their per-call transpose of every adapter
 * and without gather / scatter of the token rows. */
int trb_lora_indexed(void* y, const void* x, const void* wa, const void* wb, const void* indices,
                     int index_is_64bit, int batch, int h1, int h2, int rank, int num_adapters,
                     float scale, int dtype, int dev, void* stream);

/* Base product with the LoRA expand in the same accumulator:
 *   y[T, N] (+)= x[T, K] @ base_weight[N, K]^T  +  lora_v[T, lora_k] @ lora_b[lora_k, N]
 * on the tcgen05 tensor cores (fp32 accumulation in tensor memory, y written once).  Stands for the
 * library GEMM `x @ base_weight.t()` that opens every operator of the reference
 * (triteia/python/ops/matmul/sbmm.py:90-93, ldmm.py:72-76, lora.py:5-9) and, with lora_k > 0, for
 * the expand half of its BGMV pair (triteia/csrc/ops/bgmv_impl.cuh:141-183): lora_b is the
 * adapters' [M, r, N] tensor seen as [M * r, N] and lora_v comes from trb_lora_shrink_rows.
 * lora_k = 0 (lora_v, lora_b NULL): base product only.  accumulate != 0: y += instead of y =.
 * K % 64 == 0, N % 8 == 0, lora_k % 8 == 0; dtype TRB_F16 or TRB_BF16 for all tensors. */
int trb_base_gemm(const void* x, const void* base_weight, void* y, int num_tokens, int prob_m, int prob_k,
                  const void* lora_v, const void* lora_b, int lora_k, int accumulate, int dtype, int dev,
                  void* stream);

/* SGMV on a stacked weight tensor, on the tcgen05 tensor cores:
 *   y[s[i] : s[i + 1], :] (+)= x[s[i] : s[i + 1], :] @ w[i],   i < num_problems,
 * x [num_rows, d_in], y [num_rows, d_out], w [num_problems, d_in, d_out] row-major (the layout of the
 * Python operators' weights_A / weights_B), s int32 [num_problems + 1] on the device (a negative
 * s[0] counts as 0).  Same arithmetic as trb_sgmv / sgmv<T> (csrc/ops/sgmv.cuh:61-174: alpha = 1,
 * beta = 1 with accumulate != 0, fp32 accumulation) without the per-problem pointer array: the
 * weights of a problem are rows [i * d_in, (i + 1) * d_in) of one tensor, which one TMA descriptor
 * covers.  Called twice (shrink into v, expand into y) it is the LoRA pair of lora_sgmv
 * (triteia/python/ops/matmul/lora.py:50-105).  max_rows: an upper bound of the longest segment when
 * the caller knows one (0: num_rows); it sizes the token tile.  d_in % 8 == 0, d_out % 8 == 0,
 * num_problems <= 1024; dtype TRB_F16 or TRB_BF16. */
int trb_sgmv_stacked(void* y, const void* x, const void* w, const void* s, int num_problems, int num_rows,
                     int d_in, int d_out, int max_rows, int accumulate, int dtype, int dev, void* stream);

/* Shrink half of the indexed LoRA, written as the operand of trb_base_gemm: row b of v[B, v_cols]
 * (fp16) becomes zero except columns [id * rank, (id + 1) * rank) = scale * x[b] @ A[id], with
 * A [M, h1, rank] fp16 and id = indices[b] (int32, or int64 when index_is_64bit); ids outside
 * [0, num_adapters) leave a zero row.  v_cols >= num_adapters * rank, v_cols % 8 == 0.
 * Stands for the shrink launch of add_lora_bgmv (triteia/python/capi/punica.py:61-66,
 * triteia/csrc/ops/bgmv_impl.cuh:15-137). */
int trb_lora_shrink_rows(void* v, const void* x, const void* wa, const void* indices, int index_is_64bit,
                         int batch, int h1, int rank, int num_adapters, int v_cols, float scale, int dev,
                         void* stream);

/* SGMV: y[s[i]:s[i+1]] += x[s[i]:s[i+1]] @ w[i][layer_idx], w[i] -> [L, d_in, d_out] row-major,
 * w: device array of num_problems device pointers, s int32 [num_problems + 1].
 * Replaces sgmv<T> (csrc/ops/sgmv.h:6-9, csrc/ops/sgmv.cuh:61-174).  `tmp` is accepted for call
 * compatibility (trb_sgmv_tmp_size bytes, as csrc/ops/sgmv.cuh:48-52) and not touched. */
size_t trb_sgmv_tmp_size(int num_problems);
int trb_sgmv(void* y, const void* x, const void* w, const void* s, void* tmp, int num_problems,
             int d_in, int d_out, int layer_idx, int dtype, int dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRITEIA_B200_H_ */
