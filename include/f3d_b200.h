/* C ABI of libf3d_b200.so: the sm_100a kernels behind the Flash3D operator module
 * flash3dxfmr.lib.pshattn (reference bindings: src/f3d_frontend.cu:112-138).
 *
 * Conventions
 *  - every tensor argument is a DEVICE pointer to a contiguous row-major buffer of the stated dtype/shape;
 *    outputs are caller-allocated and written in place, exactly like the reference's at::Tensor& outputs;
 *  - sizes the reference reads from tensor shapes are passed explicitly;
 *  - `device` is the CUDA ordinal the buffers live on, `stream` a cudaStream_t (NULL = legacy default stream);
 *    the reference uses c10::cuda::getCurrentCUDAStream of the tensor's device
 *    (src/psh/batch_psh_bucket_dispatcher.cu:256);
 *  - scratch memory: entry points that need scratch beyond their arguments (PSH tile tables, the fp32 dQ accumulator of
 *    the attention backward, partial sums of the gradient reductions, the transposed operand of f3d_gemm_sm_bf16) take
 *    it from a grow-only workspace that the library keeps per (device, stream): calls on different streams use
 *    different blocks and may overlap; calls on one stream are ordered by the stream.  As for any CUDA stream, two host
 *    threads must not issue calls on the same stream concurrently.  A block that has to grow waits for its own stream
 *    only and calls cudaFree / cudaMalloc; f3d_release_workspaces frees every block (call it with the device idle).
 *    Stream capture: a call made while its stream is capturing a CUDA graph uses the stream's existing block (its
 *    address goes into the graph) and fails if that block is missing or too small, because nothing may be allocated
 *    during capture: run the same calls once on that stream first.  A block recorded in a graph is kept until
 *    f3d_release_workspaces, so the graph stays valid when later calls outgrow it;
 *  - return value 0 = ok, < 0 = error; the message is available from f3d_last_error() on the calling thread.
 *    The reference throws std::runtime_error for argument errors (src/common/runtime.h:36-86) and calls exit()
 *    on CUDA errors (src/common/runtime.h:29-34); this library returns in both cases.
 */
#ifndef F3D_B200_H
#define F3D_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define F3D_STATUS_OK 0
#define F3D_STATUS_BAD_ARGUMENT (-1)
#define F3D_STATUS_CUDA_ERROR (-2)
#define F3D_STATUS_UNSUPPORTED (-3)
#define F3D_STATUS_DEVICE (-4)

/* feature element types for the pooling / unpooling entry points */
#define F3D_DTYPE_BF16 0
#define F3D_DTYPE_FP16 1
#define F3D_DTYPE_FP32 2

/* ---- runtime state: replaces DeviceManagerSingleton (src/common/device_manager.cuh:25-64) ---- */
const char *f3d_last_error(void);
int f3d_version(void);
/* DeviceManagerSingleton::init_dev_info (src/common/device_manager.cu:73-99): checks the device is sm_100 */
int f3d_init_device(int device);
/* DeviceManagerSingleton::set_sync_stream / get_sync_stream (src/common/device_manager.cu:113-119);
 * returns the previous value */
int f3d_set_sync(int on);
int f3d_get_sync(void);
/* seed of the counter-based generator that replaces the per-device cuRAND states
 * (src/common/device_manager.cu:58-67, seed 3407) */
int f3d_set_seed(uint64_t seed);
uint64_t f3d_get_seed(void);
/* index of the calling process's first scene inside the global batch (default 0).  It is added to the scene index in
 * the random-number counter of the PSH rebalance, so that a scene-sharded run reproduces the single-process layout. */
int f3d_set_scene_base(uint32_t base);
uint32_t f3d_get_scene_base(void);
/* number of CUDA kernels this library has launched since it was loaded (benchmark bookkeeping) */
unsigned long long f3d_launch_count(void);
/* frees the library's cached scratch buffers on every device */
int f3d_release_workspaces(void);

/* ---- PSH bucketing + scatter ----
 * replaces f3d::batch_psh_scatter_pad_hash (src/psh/batch_psh_bucket_dispatcher.cu:221-326; binding
 * src/f3d_frontend.cu:120).  batch_psh_scatter and batch_psh_scatter_pad (same file :39-121, :123-219) are the
 * same call with hash_type = 3 (Z-order mod) and, for the former, pad_to_N = total_N.
 *   coord          fp16 [total_N,3]        in
 *   bucket_id      u16  [total_N]          out
 *   bucket_counter u32  [batch,num_bucket] out (final per-scene bucket sizes)
 *   bucket_offset  u32  [total_N]          out
 *   batch_sep      u32  [batch]            in  (exclusive end row of each scene = cumulative point count, i.e. the
 *                                               inclusive scan of the scene sizes; scene s covers rows
 *                                               [batch_sep[s-1], batch_sep[s]))
 *   instance_max_N                         must be >= the largest scene: it sizes the grid, and points of a scene
 *                                          beyond it would keep stale bucket ids and offsets (the reference sizes
 *                                          its grid the same way, src/psh/batch_psh_bucket_dispatcher.cu:258-262)
 *   bbox_min/max   fp16 [3]                in
 *   probe_offsets  i16  [128,3]            in
 *   cumsum_counter u32  [batch,num_bucket] out (inclusive cumsum of bucket_counter)
 *   scatter_coord  fp16 [pad_to_N,3]       out; rows [total_N,pad_to_N) are set to pad_num
 */
int f3d_batch_psh_scatter_pad_hash(
    const void *coord, void *bucket_id, void *bucket_counter, void *bucket_offset, const void *batch_sep,
    uint32_t total_N, uint32_t batch_size, uint32_t instance_max_N, uint32_t num_bucket, uint32_t bucket_divisor,
    uint32_t bucket_size, uint32_t num_vox, const void *bbox_min, const void *bbox_max, const void *probe_offsets,
    void *cumsum_counter, void *scatter_coord, uint32_t pad_to_N, float pad_num, uint32_t hash_type,
    int device, void *stream);

/* Same operation and arguments as f3d_batch_psh_scatter_pad_hash, for callers that may not allocate device memory
 * (hosts whose GPU memory belongs entirely to another allocator, or loops that cannot take the device-wide
 * synchronisation of cudaMalloc / cudaFree).  It has no counterpart in the reference.  The scratch tables live in a
 * fixed 4 MiB device array inside the library (held on every GPU that loads it); the call performs no cudaMalloc,
 * cudaFree or other allocating call.  Limits: the batch must satisfy
 *     3*B*T*(NB+1) + 5*B*(NB+1) + 2*B*T + ceil(total_N / 2) <= 1,048,576   with B = batch_size, NB = num_bucket,
 *     T = ceil(instance_max_N / tile), tile = 2048, doubled (up to 16384) while the sum does not fit (batches of
 *     fewer than 148 tiles take tiles down to 256 points while the sum still fits),
 * otherwise F3D_STATUS_UNSUPPORTED is returned (8 scans of 120,000 points with 256 buckets need 855k words at
 * tile 2048; the last term holds one 16-bit key per point).
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and sets a kernel attribute;
 * with the driver's lazy module loading that first call is also where the library's code and the array itself are
 * brought onto the device, so the no-allocation guarantee holds from the second call on: make one warm-up call per
 * device at start-up, outside any stream capture.  All calls share the array: calls that overlap on one GPU race and
 * must be serialised by the caller.  The sync_stream switch (f3d_set_sync) is honoured as in the regular entry point. */
int f3d_batch_psh_scatter_pad_hash_noalloc(
    const void *coord, void *bucket_id, void *bucket_counter, void *bucket_offset, const void *batch_sep,
    uint32_t total_N, uint32_t batch_size, uint32_t instance_max_N, uint32_t num_bucket, uint32_t bucket_divisor,
    uint32_t bucket_size, uint32_t num_vox, const void *bbox_min, const void *bbox_max, const void *probe_offsets,
    void *cumsum_counter, void *scatter_coord, uint32_t pad_to_N, float pad_num, uint32_t hash_type,
    int device, void *stream);

/* ---- scoreboard check of a finished bucketing (host code, no kernel) ----
 * replaces f3d::batch_bucket_sanitizer_cpu (src/psh/bucket_sanitizer_cpu.cpp:92-176; binding src/f3d_frontend.cu:133;
 * call site tests/test_psh.py:127-129).  Every pointer is a HOST pointer (the reference moves each tensor to the CPU
 * before it reads it, :104-110):
 *   bucket_id          u16 [total_N]                          in
 *   bucket_counter     u32 [batch,num_bucket]                 in
 *   bucket_offset      u32 [total_N]                          in
 *   offset_check_table i8  [batch,num_bucket,table_slots]     in/out: += 1 at every point's (scene, bucket, offset)
 *   bucket_residual    u32 [batch,num_bucket]                 in/out: -= 1 per point of the bucket (a copy of
 *                                                             bucket_counter ends at zero)
 *   batch_sep          u32 [batch]                            in
 *   offset_maxcnt      u32 [batch]                            in  (largest bucket count of each scene)
 * Returns F3D_STATUS_BAD_ARGUMENT, with the position in f3d_last_error(), for a bucket id >= num_bucket, an offset >=
 * offset_maxcnt of its scene, or a slot below a bucket's count that was not marked exactly once (the reference throws
 * std::runtime_error with the same text). */
int f3d_batch_bucket_sanitizer_cpu(
    const void *bucket_id, const void *bucket_counter, const void *bucket_offset, void *offset_check_table,
    void *bucket_residual, const void *batch_sep, const void *offset_maxcnt, uint32_t total_N, uint32_t batch_size,
    uint32_t num_bucket, uint32_t table_slots);

/* ---- sub-bucket construction + feature pooling ----
 * replaces f3d::batch_subbuck_reduce (src/psh/batch_subbuck_pooling_dispatcher.cu:35-144; binding
 * src/f3d_frontend.cu:127): local_subbuck_ker followed by reduce_feat_ker.
 *   scattered_coord   fp16 [total_N,3]                 in
 *   scattered_feat    feat_dtype [>= total_N, feat_dim] in
 *   batch_sep         u32 [batch]                      in
 *   bbox_min/max      fp16 [3]                         in  (accepted for signature parity; the hash normalises
 *                                                          with each 1024-point block's own bounding box)
 *   subbuck_id        u32 [total_N]                    out (row inside the scene's reduced rows)
 *   subbuck_off       u16 [total_N]                    out (slot inside the sub-bucket)
 *   reduced_batch_sep u32 [batch]                      in  (inclusive end of each scene's reduced rows)
 *   reduced_coord     fp16 [reduced_rows,3]            out (mean member coordinate; rows >= unpool_rows := 0)
 *   reduced_feat      feat_dtype [reduced_rows,feat_dim] out (rows >= unpool_rows := 0)
 *   unpool_ind        u32 [unpool_rows,subbuck_size]   out (slots of short sub-buckets get total_N + 3, the value the
 *                                                          reference pre-fills with; a pre-filled table is accepted)
 *   red_op            0 mean, 1 sum, 2 min, 3 max
 */
int f3d_batch_subbuck_reduce(
    const void *scattered_coord, const void *scattered_feat, const void *batch_sep, uint32_t total_N,
    uint32_t batch_size, uint32_t instance_max_N, uint32_t subbuck_size, uint32_t num_vox, const void *bbox_min,
    const void *bbox_max, void *subbuck_id, void *subbuck_off, const void *reduced_batch_sep, void *reduced_coord,
    void *reduced_feat, void *unpool_ind, uint32_t unpool_rows, uint32_t reduced_rows, uint32_t feat_dim,
    int feat_dtype, uint32_t hash_type, uint32_t red_op, int device, void *stream);

/* replaces f3d::batch_subbuck_reduce_backward (src/psh/batch_subbuck_pooling_bwd_dispatcher.cu:26-85; binding
 * src/f3d_frontend.cu:128).  grad_input_feat must be zero-initialised by the caller
 * (flash3dxfmr/layers/pooling.py:102); only rows referenced by unpool_ind are written. */
int f3d_batch_subbuck_reduce_backward(
    const void *grad_red_feat, const void *input_feat, const void *unpool_ind, void *grad_input_feat, uint32_t total_N,
    uint32_t unpool_rows, uint32_t feat_dim, int feat_dtype, uint32_t subbuck_size, uint32_t red_op, int device,
    void *stream);

/* replaces f3d::additive_unpool_fwd (src/psh/additive_unpool_dispatcher.cu:26-79; binding
 * src/f3d_frontend.cu:123): up[r] = res[r] + down[i] for every valid r = unpool_ind[i, s].
 * Rows [covered_rows, up_rows) of up_add_feat, which no index refers to (tail padding), are set to zero; pass
 * covered_rows = up_rows to leave them untouched as the reference does. */
int f3d_additive_unpool_fwd(
    const void *res_feat, const void *down_feat, void *up_add_feat, const void *unpool_ind, uint32_t up_rows,
    uint32_t unpool_rows, uint32_t covered_rows, uint32_t feat_dim, int feat_dtype, uint32_t subbuck_size, int device,
    void *stream);

/* replaces f3d::additive_unpool_bwd (src/psh/additive_unpool_dispatcher.cu:81-134; binding
 * src/f3d_frontend.cu:124): grad_res[r] = g[r]; grad_down[i] = sum_s g[unpool_ind[i,s]]. */
int f3d_additive_unpool_bwd(
    void *grad_res, void *grad_down, const void *grad_up_added, const void *unpool_ind, uint32_t up_rows,
    uint32_t unpool_rows, uint32_t feat_dim, int feat_dtype, uint32_t subbuck_size, int device, void *stream);

/* ---- bucketed self-attention backward ----
 * provides f3d::buck_swin_bwd, declared at src/f3d_frontend.cu:94-97 and called by
 * flash3dxfmr/layers/buck_swin.py:91; absent from the reference snapshot like the forward.  Semantics:
 * tests/test_attn_bwd.py:24-27,54-62,79-441.
 *   Q, K, V, O, dO  bf16 [B,L,H,D]   in  (O and LSE may come from any forward implementation)
 *   LSE             fp32 [B,L,H]     in
 *   Delta           fp32 [B,L,H]     out  rowsum(dO * O)
 *   dQ, dK, dV      bf16 [B,L,H,D]   out  (dQ is written for every token - zero for buckets no scope lists; dK, dV
 *                                          only for listed buckets: zero-fill them beforehand, as the reference's
 *                                          BuckSwinBwdBuffers does, when the table leaves buckets out)
 * A bucket may appear in at most one scope (the reference's scope plans are partitions,
 * flash3dxfmr/psh/bucket_scope.py:58-140); with a bucket listed twice the result is undefined.
 * Windows above 512 tokens use an fp32 scratch of B*L*H*D elements for the dQ reduction (library workspace, below);
 * smaller windows at D <= 32 keep dQ in tensor memory and need none. */
int f3d_buck_swin_bwd(const void *Q, const void *K, const void *V, const void *O, const void *dO, const void *LSE,
                      void *Delta, void *dQ, void *dK, void *dV, const void *scope_buckets, int B, int L, int H, int D,
                      int num_scopes, int scope_size, uint32_t bucket_size, int device, void *stream);

/* reads and clears the device status word: kernels that wait on mbarriers give up after a bounded time and record
 * the waiting site there; returns F3D_STATUS_DEVICE if a wait was abandoned since the last call (synchronises). */
int f3d_device_status(int device);

/* ---- per-token projection GEMM ----
 * replaces the cuBLAS GEMMs behind nn.Linear in BucketSwinAttentionModule (flash3dxfmr/layers/buck_swin.py:159,163,
 * 185-194): C = A . W^T (+ bias) (+ residual), bf16 operands, fp32 accumulation on tcgen05 tensor cores.
 *   A        bf16 [M,K]   in   (activations, row-major)
 *   W        bf16 [N,K]   in   (nn.Linear weight layout)
 *   bias     fp32 [N]     in   or NULL
 *   residual bf16 [M,N]   in   or NULL (added after the bias; nsplit must be 1)
 *   C        bf16         out  nsplit matrices [M, N/nsplit], stored one after another (nsplit = 3 writes Q, K and V
 *                              as three contiguous [M, H*D] matrices)
 *   epilogue 0 none, 1 GELU(tanh), 2 SwiGLU: W = [gate; up] (N = 2*F rows), C[M,F] = silu(gate) * up
 * K, N/nsplit must be multiples of 8; pointers 16-byte aligned. */
int f3d_linear_bf16(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N, int K,
                    int nsplit, int epilogue, int device, void *stream);

/* f3d_linear_bf16 with the element type as an argument: dtype F3D_DTYPE_BF16 or F3D_DTYPE_FP16 for A, W, residual and
 * C (bias stays fp32, accumulation fp32).  The reference states its CPU-runnable configuration in fp16 features; this
 * entry point and f3d_buck_swin_fwd_dtype serve it (forward only). */
int f3d_linear_dtype(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N, int K,
                     int nsplit, int epilogue, int dtype, int device, void *stream);

/* f3d_linear_dtype with a LayerNorm folded in and / or row sums of the output written out.  In the reference every
 * projection of a transformer block is preceded by a LayerNorm kernel of its own (te.LayerNorm / LayerNormMLP,
 * flash3dxfmr/layers/stage.py:95, flash3dxfmr/layers/elem_wise.py:22-26); here the chain
 * projection -> LayerNorm -> projection runs as two GEMMs and nothing else:
 *   stats_out  fp32 [M,2] or NULL: (sum, sum of squares) of every output row (after bias and residual, before the
 *              rounding to the output type), added up by the epilogue in a fixed order (same bits on every run for
 *              N <= 512); needs nsplit == 1 and no SwiGLU
 *   ln_stats   fp32 [M,2] or NULL: (sum, sum of squares) of every row of A over its K channels - the stats_out of the
 *              GEMM that produced A, or f3d_row_stats_bf16.  With it the call computes LayerNorm(A) W0^T + b0 for a
 *              LayerNorm with weight gamma and bias beta, given W = W0 diag(gamma) (same element type as A),
 *              ln_colsum fp32 [N] = row sums of that scaled W as stored, bias fp32 [N] = b0 + W0 beta, ln_eps. */
int f3d_linear_fused(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N, int K,
                     int nsplit, int epilogue, int dtype, const void *ln_stats, const void *ln_colsum, float ln_eps,
                     void *stats_out, int device, void *stream);

/* stats fp32 [rows,2] = (sum, sum of squares) over the C channels of every row of x bf16 [rows, C]: the ln_stats input
 * of f3d_linear_fused for rows that no GEMM of this library produced.  C a multiple of 8, <= 2048. */
int f3d_row_stats_bf16(const void *x, void *stats, uint32_t rows, uint32_t C, int device, void *stream);

/* replaces f3d::gemm_sm_bf16 (src/psh/gemm_dispatcher.cu:26-80; binding src/f3d_frontend.cu:135): O[M,N] = A[M,K] . B[K,N],
 * bf16 in/out, fp32 accumulation; synchronises the stream like the reference (:77).  Any M; N, K multiples of 8. */
int f3d_gemm_sm_bf16(const void *A, const void *B, void *O, int M, int N, int K, int device, void *stream);

/* ---- bucketed self-attention forward ----
 * provides f3d::buck_swin_fwd, declared at src/f3d_frontend.cu:90-92 and called by
 * flash3dxfmr/layers/buck_swin.py:57; the reference snapshot holds neither its kernel nor its binding
 * (src/f3d_frontend.cu:136 is commented out).  Semantics: tests/test_attn_fwd.py:295-452.
 *   Q, K, V        bf16 [B,L,H,D]          in
 *   O              bf16 [B,L,H,D]          out (tokens of buckets no scope lists are left untouched)
 *   LSE            fp32 [B,L,H]            out (natural-log softmax normaliser)
 *   scope_buckets  u32  [num_scopes,scope_size]  in: each row lists the buckets that attend to each other
 * D in {16,32,64,128}; bucket_size a multiple of 128; L a multiple of bucket_size. */
int f3d_buck_swin_fwd(const void *Q, const void *K, const void *V, void *O, void *LSE, const void *scope_buckets,
                      int B, int L, int H, int D, int num_scopes, int scope_size, uint32_t bucket_size,
                      int device, void *stream);

/* f3d_buck_swin_fwd with the element type of Q, K, V, O as an argument (F3D_DTYPE_BF16 or F3D_DTYPE_FP16; the
 * probabilities that enter the second product are rounded to the same type).  Forward only: f3d_buck_swin_bwd takes
 * bf16. */
int f3d_buck_swin_fwd_dtype(const void *Q, const void *K, const void *V, void *O, void *LSE, const void *scope_buckets,
                            int B, int L, int H, int D, int num_scopes, int scope_size, uint32_t bucket_size, int dtype,
                            int device, void *stream);

/* LayerNorm over the last dimension of bf16 [rows, C] with fp32 weight/bias [C] and an optional exact GELU.
 * Stands in for the te.LayerNorm / nn.LayerNorm steps of XFMR and the pooling wrappers
 * (flash3dxfmr/layers/stage.py:67,95; flash3dxfmr/layers/hourglass.py:76-79).  C a multiple of 8, <= 2048. */
int f3d_layernorm_bf16(const void *x, const void *weight, const void *bias, void *y, uint32_t rows, uint32_t C, float eps,
                       int gelu, int device, void *stream);

/* Backward of f3d_layernorm_bf16 without GELU: grad_x bf16 [rows, C], grad_weight / grad_bias fp32 [C] from x and grad_out
 * (bf16 [rows, C]) and the fp32 weight.  The reference gets this from TransformerEngine's / torch's LayerNorm backward
 * (flash3dxfmr/layers/stage.py:67,95).  Row sums are added in a fixed order (same bits every run).  C a multiple of 8,
 * <= 1024. */
int f3d_layernorm_bwd_bf16(const void *x, const void *grad_out, const void *weight, void *grad_x, void *grad_weight,
                           void *grad_bias, uint32_t rows, uint32_t C, float eps, int device, void *stream);

/* Backward of the SwiGLU epilogue out = silu(gate) * up: pre_act bf16 [rows, 2F] = [gate | up] (the fc1 GEMM's result
 * before the activation), grad_out bf16 [rows, F] -> grad_pre_act bf16 [rows, 2F].  The reference's MLP is
 * TransformerEngine's LayerNormMLP with activation "swiglu" (flash3dxfmr/layers/elem_wise.py); F a multiple of 8. */
int f3d_swiglu_bwd_bf16(const void *pre_act, const void *grad_out, void *grad_pre_act, uint64_t rows, uint32_t F, int device,
                        void *stream);

/* Backward of out = gelu(y): grad_pre_act = grad_out * gelu'(pre_act), all bf16 with `elems` elements (a multiple of 8).
 * tanh_form = 0: the exact form (error function) of the LayerNorm + GELU in the reference's pooling / unpooling wrappers
 * (flash3dxfmr/layers/hourglass.py:101-103, 181-185), whose backward the reference takes from torch autograd;
 * tanh_form = 1: the tanh form that the GELU epilogue of f3d_linear_bf16 computes. */
int f3d_gelu_bwd_bf16(const void *pre_act, const void *grad_out, void *grad_pre_act, uint64_t elems, int tanh_form, int device,
                      void *stream);

/* Bias gradient: out fp32 [C] = column sums of x bf16 [rows, C], added in a fixed order.  C a multiple of 8. */
int f3d_colsum_bf16(const void *x, void *out, uint64_t rows, uint32_t C, int device, void *stream);

/* Coordinate embedding out = W x + b: fp16 coordinates [rows, 3], fp32 weight [C, 3] and bias [C], bf16 out [rows, C].
 * Stands in for the te.Linear(3, emb_dim) of PSH3DCoordEmbedding (flash3dxfmr/layers/psh_ops.py:62,77).  C a multiple
 * of 8, <= 2048. */
int f3d_coord_embed_bf16(const void *coords, const void *weight, const void *bias, void *out, uint32_t rows, uint32_t C,
                         int device, void *stream);

/* Parameter gradients of the coordinate embedding: grad_weight fp32 [C, 3] = grad_out^T coords and grad_bias fp32 [C]
 * (may be NULL) = column sums of grad_out, for fp16 coords [rows, 3] and bf16 grad_out [rows, C]; sums added in a fixed
 * order.  The reference gets them from te.Linear's backward (flash3dxfmr/layers/psh_ops.py:62,77). */
int f3d_coord_embed_bwd(const void *coords, const void *grad_out, void *grad_weight, void *grad_bias, uint32_t rows, uint32_t C,
                        int device, void *stream);

/* Weight and bias gradient of a projection y = x W^T + b: grad_weight fp32 [N, K] = grad_out^T x and, when grad_bias is
 * not NULL, grad_bias fp32 [N] = column sums of grad_out, for grad_out bf16 [M, N] and x bf16 [M, K] (both dense).  One
 * pass over grad_out and x on the tensor cores (neither is transposed in memory), sums over row slabs added in a fixed
 * order.  N a multiple of 8; K = 32 or a multiple of 64. */
int f3d_linear_wgrad_bf16(const void *grad_out, const void *x, void *grad_weight, void *grad_bias, int M, int N, int K,
                          int device, void *stream);

/* Sum of slice products C[M, N] = sum_s A[s] W[s]^T (+ bias) (+ residual): A bf16 [ksplit, M, K], W bf16 [ksplit, N, K],
 * both dense.  One GEMM whose k-blocks walk the slices; it is the input gradient of a projection that wrote its output as
 * separate matrices (the Q, K, V layout of f3d_linear_bf16 with nsplit = 3: grad_x = sum_s grad[s] W_s), without first
 * interleaving the three gradients.  K a multiple of 8. */
int f3d_linear_ksplit_bf16(const void *A, const void *W, const void *bias, const void *residual, void *C, int M, int N, int K,
                           int ksplit, int device, void *stream);

/* Raw scan records to operator inputs: records fp32 [rows, point_dim] (x, y, z, then intensity / ring / time; the
 * layout of KITTI and nuScenes .bin files, point_dim 3..6) -> coords fp16 [rows, 3] (round to nearest even) and, when
 * extra is not NULL, extra fp32 [rows, point_dim - 3].  One pass on the device in place of the cast, slice and copy of
 * collate_coords_flat_sep (flash3dxfmr/psh/batching.py:13-28). */
int f3d_collate_points_f32(const void *records, void *coords, void *extra, uint64_t rows, uint32_t point_dim, int device,
                           void *stream);

/* Scatter index of the bucket order (the part of batch_psh_cumsum_scatter_feat_index_postpad_ker the reference wrote,
 * src/psh/batch_psh_bucket.cuh:617-753, plus its inverse): from the outputs of f3d_batch_psh_scatter - bucket_id u16 [N],
 * bucket_offset u32 [N], cumsum_counter u32 [B, num_bucket] (inclusive) and batch_sep u32 [B] (cumulative point counts: exclusive scene ends) -
 * out2in u32 [pad_to_N]: out2in[row in bucket order] = input row, rows [total_N, pad_to_N) = total_N + 3 (the
 * reference's padding mark, batch_psh_bucket.cuh:667); in2out u32 [total_N] (may be NULL): in2out[input row] = row in
 * bucket order. */
int f3d_scatter_index(const void *bucket_id, const void *bucket_offset, const void *cumsum_counter, const void *batch_sep,
                      void *out2in, void *in2out, uint32_t total_N, uint32_t batch_size, uint32_t num_bucket,
                      uint32_t pad_to_N, int device, void *stream);

/* Row gather out[i, :] = src[index[i], :] for i < rows_out; rows whose index is >= rows_src (the padding mark) are
 * zero.  Rows are row_bytes bytes (a multiple of 4) of any element type.  With out2in it scatters input features into
 * bucket order (what scattered_feat of batch_psh_bucket.cuh:627 was meant to receive), with in2out it brings results
 * back to the input order; each is the other's backward. */
int f3d_gather_rows(const void *src, const void *index, void *out, uint64_t rows_out, uint32_t rows_src, uint32_t row_bytes,
                    int device, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* F3D_B200_H */
