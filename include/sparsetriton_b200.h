/*
 * libsparsetriton_b200 -- C ABI of the B200 (sm_100a) sparse-convolution hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*,
 * i.e. a cudaStream_t; NULL = legacy default stream) and returns an int status:
 *     0  ST_OK
 *    <0  argument / support error detected on the host before any launch (table below)
 * Conditions detected on the device (hash table full, output buffer too small) are written to a
 * caller-supplied int32 status word in device memory; the bits are listed at ST_DEV_*.
 * No entry point allocates or frees memory: scratch is passed in by the caller, sized by the
 * matching *_workspace_bytes() call.  All work is enqueued on the given stream; nothing here
 * synchronises.
 *
 * Each declaration names the function of ptj0225/SparseTriton it stands in for
 * (path:line inside that project).  The reference has no FFI of its own -- its kernels are
 * Triton programs called from Python -- so "replaces" means: the Python callable of the same
 * role calls this entry point instead of launching the Triton kernel.
 *
 * Layouts
 *   coordinates  (N,4) row-major, columns (batch, x, y, z); int16 (ST_I16) or int32 (ST_I32);
 *                every value must lie in [0, 65535] to be representable in a key
 *   hash table   keys  int64[capacity], -1 = empty, else batch<<48 | x<<32 | y<<16 | z
 *                vals  int32[capacity], row index of the key, -1 = empty
 *   offsets      (K,3) int32 in HOST memory (copied into the launch parameters), K <= 343
 *   neighbour map  int32 (N_out, K) row-major, -1 = no neighbour  (the reference's layout)
 *   features     (N, C) row-major, fp32 / fp16 / bf16; weights (K, Cin, Cout) row-major, same dtype
 */
#ifndef SPARSETRITON_B200_H
#define SPARSETRITON_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ST_OK 0
#define ST_ERR_ARG (-1)         /* null pointer, negative size, K out of range ... */
#define ST_ERR_DTYPE (-2)       /* unknown dtype code */
#define ST_ERR_WORKSPACE (-3)   /* workspace too small or misaligned */
#define ST_ERR_CUDA (-4)        /* a launch was rejected; st_last_error_string() has the text */
#define ST_ERR_UNSUPPORTED (-5) /* shape outside what the kernels handle */

#define ST_DEV_TABLE_FULL 1     /* an insert ran out of probes: capacity too small */
#define ST_DEV_OUT_OVERFLOW 2   /* more output rows than the caller's buffer holds */
#define ST_DEV_BAD_INDEX 4      /* a map entry pointed outside the feature matrix (debug checks) */
#define ST_DEV_TIMEOUT 8        /* a bounded wait inside a tensor-core kernel expired; the kernel unwound */

#define ST_I16 0
#define ST_I32 1

#define ST_F32 0                /* fp32 storage; tensor-core kernels multiply in tf32 */
#define ST_F16 1
#define ST_BF16 2

#define ST_MAX_KVOL 343

/* Library revision (monotonic integer). */
int st_version(void);
/* Text of the last host-side error of the calling thread. */
const char* st_last_error_string(void);
/* Number of kernels this library has enqueued in this process so far. */
long long st_launch_count(void);
/* Sticky status of the tensor-core kernels on the current device: out4 (HOST memory, 4 x int32) =
 * {ST_DEV_* flags, id of the wait that expired, block index, reserved}.  Synchronises the stream. */
int st_device_status(int32_t* out4, void* stream);

/* The same copy without the synchronisation: out4 (PINNED host memory) holds the four words once the stream has
 * passed this point.  Lets a caller fold the check into a wait it makes anyway.  No reference counterpart. */
int st_device_status_enqueue(int32_t* pinned_out4, void* stream);

/* Clears the sticky status word of the current device (stream-ordered).  No reference counterpart. */
int st_device_status_clear(void* stream);
/* 1 if the tcgen05 (tensor-core) kernels can serve this conv shape, else 0 (SIMT kernels used). */
int st_conv_uses_tensor_cores(int dtype, int cin, int cout);
/* Process-wide switch (default on).  With 0 every product runs on the CUDA-core kernels; used to
 * cross-check the tensor-core kernels and to get exact-fp32 arithmetic for fp32 features. */
int st_set_tensor_cores(int enable);
/* Process-wide switch (default on): products over a tile plan use the kernels fed by TMA (tile::gather4);
 * when off, or when a tensor's base or row pitch is not 16-byte aligned, their cp.async forms run over
 * the same plan.  Results are identical. */
int st_set_tma(int enable);

/* 1 (default): the planned weight gradient copies dY into tile order once and loads its tiles as dense boxes; 0: it
 * gathers the rows of every tile through the row order (the earlier form, kept for comparison).  No reference counterpart. */
int st_set_dense_tiles(int enable);

/* ---------------------------------------------------------------- hash table ------------- */

/* Fill keys and vals with -1.
 * Replaces the two torch.full(-1) fills of HashTable.__init__, sparsetriton/utils/hash.py:428-429. */
int st_hash_clear(int64_t* keys, int32_t* vals, int64_t capacity, void* stream);

/* Insert n coordinates; value = row index; a repeated coordinate keeps its largest row.
 * Replaces HashTable.insert -> build_hash_table_kernel, sparsetriton/utils/hash.py:516-544, 193-258.
 * status: device int32, ST_DEV_TABLE_FULL is OR-ed in if some key found no slot, ST_DEV_BAD_INDEX if a
 * coordinate has a value outside [0, 65535] (that row is left out of the table). */
int st_hash_build(const void* coords, int64_t n, int coord_dtype, int64_t* keys, int32_t* vals,
                  int64_t capacity, int32_t* status, void* stream);

/* out[i] = row of coords[i] or -1.
 * Replaces HashTable.query -> query_hash_table_kernel, sparsetriton/utils/hash.py:546-580, 261-366. */
int st_hash_query(const void* coords, int64_t m, int coord_dtype, const int64_t* keys, const int32_t* vals,
                  int64_t capacity, int32_t* out, void* stream);

/* ---------------------------------------------------------------- output coordinates ----- */

/* Scratch needed by st_outcoords_count/_write for n inputs and K offsets. */
int64_t st_outcoords_workspace_bytes(int64_t n, int K, int stride, int transposed);

/* Pass 1 of the output-coordinate build of a strided (transposed = 0) or transposed conv:
 * enumerate candidates  in+off (kept if divisible by stride on every axis, then divided)  or
 * in*stride+off (transposed; batch column unscaled), drop those outside [0,new_shape), dedupe
 * keeping the candidate with the smallest flat index n*K+k, and write the number of survivors
 * to *n_out (device or pinned-host int64).
 * Replaces _build_out_coords_normal / _build_out_coords_transposed with expand_coords_kernel,
 * mask_spatial_range and filter_unique_kernel: nn/functional/conv/kmap.py:213-444, 11-97,
 * utils/spatial/tile.py:6-84.
 *
 * batch_bound (all three passes, the same value): the number of samples the batch holds, if the caller knows it,
 * else 0.  With it, and an output grid of at most 2^29 cells over all samples whose bitmaps fit the workspace, the
 * coordinates are deduplicated by direct addressing (one bit per cell, ranks by popcount) instead of through a
 * hash table: same results, but every structure then lives in L2.  Rows whose batch index is outside
 * [0, batch_bound) are then skipped and ST_DEV_BAD_INDEX is OR-ed into *status. */
int st_outcoords_count(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K,
                       int stride, int transposed, const int32_t* new_shape_host, int batch_bound, void* workspace,
                       int64_t workspace_bytes, int64_t* n_out, int32_t* status, void* stream);

/* Pass 2: write the surviving coordinates, ordered by first occurrence (n-major, k-minor), into
 * out_coords (same integer type as coords, out_capacity rows).  Must follow st_outcoords_count on
 * the same stream with the same arguments and workspace. */
int st_outcoords_write(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K,
                       int stride, int transposed, const int32_t* new_shape_host, int batch_bound, void* workspace,
                       int64_t workspace_bytes, void* out_coords, int64_t out_capacity, int32_t* status,
                       void* stream);

/* Pass 3 (optional): the neighbour map of the same convolution, nbr (n_out, K) int32, produced by a
 * scatter over the surviving candidates -- candidate (n, k) lands on output row o, so nbr[o,k] = n --
 * instead of n_out*K probes of the input table.  Equals st_map_build on the written coordinates.
 * in_shape_host: the input grid (inputs outside it get no map entry, as with the probing form).
 * Must follow st_outcoords_write on the same stream with the same arguments and workspace.
 * Replaces compute_neighbor_indices for strided / transposed layers, nn/functional/conv/conv.py:12-75. */
int st_outcoords_map(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K, int stride,
                     int transposed, const int32_t* new_shape_host, const int32_t* in_shape_host, int batch_bound,
                     void* workspace, int64_t workspace_bytes, int32_t* nbr, int64_t n_out, void* stream);

/* ---------------------------------------------------------------- neighbour map ---------- */

/* nbr[o,k] = row of (batch, out*lookup_stride - off[k]) if inside [0,lookup_shape) and present.
 * Replaces compute_neighbor_indices, nn/functional/conv/conv.py:12-75. */
int st_map_build(const void* out_coords, int64_t n_out, int coord_dtype, const int32_t* offsets_host, int K,
                 int lookup_stride, const int32_t* lookup_shape_host, const int64_t* keys, const int32_t* vals,
                 int64_t capacity, int32_t* nbr, void* stream);

/* The same map for a submanifold layer, where the queried coordinates are the rows the table was built
 * from (row r has value r, or a larger row with the same coordinate), the stride is 1 and the offsets come
 * in opposite pairs (off[K-1-k] = -off[k], K odd; checked): only offsets 0..K/2 are probed, the rest follows
 * from "i is o's neighbour at k  <=>  o is i's neighbour at K-1-k".  Same result as st_map_build, entry for
 * entry, including duplicate and out-of-grid coordinates.  *asymmetric_rows (device int32, may be NULL)
 * receives the number of rows the table does not return for their own coordinate; when it is 0 the map
 * is symmetric and st_conv_dgrad_mirrored may be used. */
int st_map_build_symmetric(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K,
                           const int32_t* lookup_shape_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                           int32_t* nbr, int32_t* asymmetric_rows, void* stream);

/* inv[i,k] = o for every nbr[o,k] = i >= 0, -1 elsewhere (inv is (n_in,K) and is fully written).
 * No counterpart in the reference, whose dgrad scatters with atomics
 * (funcs/implicit_precomputed_gemm.py:129-177); this is the map its gather-form dgrad reads. */
int st_map_invert(const int32_t* nbr, int64_t n_out, int K, int64_t n_in, int32_t* inv, void* stream);

/* A row order for the convolution entry points below: order (n_rows int32) <- the rows of a
 * neighbour map (forward or inverse) sorted, stably, by which of their K offsets are occupied.
 * The tensor-core kernels work on tiles of 128 rows and skip an offset only when no row of the
 * tile has a neighbour there; walking the rows in this order makes tiles share their occupied
 * offsets (2-4x fewer tile x offset steps on surface-like data).  Deterministic.
 * No counterpart in the reference (its kernels mask per element inside every tile). */
int64_t st_map_row_order_workspace_bytes(int64_t n_rows, int K);
int st_map_row_order(const int32_t* nbr, int64_t n_rows, int K, int32_t* order, void* workspace,
                     int64_t workspace_bytes, void* stream);

/* Tile plan of a neighbour map for the tensor-core kernels: the map re-laid tile by tile (128 rows
 * in the walking order) and offset by offset, so that the 128 source rows of one tile x offset step
 * are one 512-byte line, plus one bit per tile and offset saying whether the step has any neighbour:
 *   tmap [(tile*K + k)*128 + r] = nbr[order[tile*128 + r], k]   (ceil(n_rows/128)*K*128 int32)
 *   tmask[tile*ceil(K/32) + k/32] bit k%32                      (ceil(n_rows/128)*ceil(K/32) uint32)
 * sort_rows != 0 first computes `order` as st_map_row_order() does (workspace as for that call);
 * sort_rows == 0 plans the natural order (order, workspace unused).
 * No counterpart in the reference. */
int64_t st_map_plan_workspace_bytes(int64_t n_rows, int K);
int st_map_plan(const int32_t* nbr, int64_t n_rows, int K, int sort_rows, int32_t* order, int32_t* tmap,
                uint32_t* tmask, void* workspace, int64_t workspace_bytes, void* stream);

/* The tile plan of the INVERSE of a map, straight from the forward map: what st_map_invert followed by
 * st_map_plan(sort_rows = 1) gives (identical arrays), without writing or re-reading the (N_in, K) inverse.
 * K <= 32.  Used by the feature gradient of strided / transposed layers. */
int64_t st_map_plan_inverse_workspace_bytes(int64_t n_in, int K);
int st_map_plan_inverse(const int32_t* nbr, int64_t n_out, int K, int64_t n_in, int32_t* order, int32_t* tmap,
                        uint32_t* tmask, void* workspace, int64_t workspace_bytes, void* stream);

/* Scratch for st_map_pairs_count/_write. */
int64_t st_map_pairs_workspace_bytes(int64_t n_out, int K);
/* Number of valid entries of a neighbour map -> *n_pairs (device or pinned-host int64). */
int st_map_pairs_count(const int32_t* nbr, int64_t n_out, int K, void* workspace, int64_t workspace_bytes,
                       int64_t* n_pairs, void* stream);
/* The map as (in_idx, out_idx, offset) int32 triples in (out_idx, offset) order; follows _count.
 * No counterpart in the reference (its map stays dense); used for pair statistics and parity. */
int st_map_pairs_write(const int32_t* nbr, int64_t n_out, int K, void* workspace, int64_t workspace_bytes,
                       int32_t* triples, int64_t capacity, int32_t* status, void* stream);

/* ---------------------------------------------------------------- convolution ------------ */

/* Scratch for the three products with a stored map (max over fwd/dgrad/wgrad). */
int64_t st_conv_workspace_bytes(int dtype, int64_t n_in, int64_t n_out, int K, int cin, int cout);

/* Y[o,:] = sum_k X[nbr[o,k],:] . W[k]      fp32 accumulation, Y in the feature dtype.
 * Replaces ConvPrecomputedNeighborGEMM.forward -> precomputed_fwd_kernel,
 * funcs/implicit_precomputed_gemm.py:237-276, 64-126. */
int st_conv_fwd(int dtype, const void* X, const void* W, const int32_t* nbr, void* Y, int64_t n_in,
                int64_t n_out, int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);

/* dX[i,:] = sum_k dY[inv[i,k],:] . W[k]^T  (gather form over the inverse map; deterministic).
 * Replaces precomputed_bwd_feat_kernel, funcs/implicit_precomputed_gemm.py:278-304, 129-177. */
int st_conv_dgrad(int dtype, const void* dY, const void* W, const int32_t* inv, void* dX, int64_t n_in,
                  int64_t n_out, int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);

/* dW[k] = sum_o X[nbr[o,k],:]^T . dY[o,:]  split over (offset, row chunk) into fp32 partials that
 * a second kernel reduces in a fixed order.
 * Replaces precomputed_bwd_weight_kernel, funcs/implicit_precomputed_gemm.py:306-324, 180-230. */
int st_conv_wgrad(int dtype, const void* X, const void* dY, const int32_t* nbr, void* dW, int64_t n_in,
                  int64_t n_out, int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);

/* The three products over a map that comes with a tile plan from st_map_plan() (of the map they are
 * given: the forward map for fwd and wgrad, the inverse map for dgrad).  row_order, tmap and tmask
 * may each be NULL: without tmap/tmask the kernels read `nbr` itself, without row_order they walk
 * the rows in natural order.  st_conv_dgrad_planned also accepts inv = NULL when the plan is given and
 * st_conv_uses_tensor_cores(dtype, cout, cin) holds (the plan from st_map_plan_inverse).  Forward and feature-gradient results do not depend on the order; the
 * weight gradient adds its rows in that order (still the same from run to run). */
int st_conv_fwd_planned(int dtype, const void* X, const void* W, const int32_t* nbr, const int32_t* row_order,
                        const int32_t* tmap, const uint32_t* tmask, void* Y, int64_t n_in, int64_t n_out, int K,
                        int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);
int st_conv_dgrad_planned(int dtype, const void* dY, const void* W, const int32_t* inv, const int32_t* row_order,
                          const int32_t* tmap, const uint32_t* tmask, void* dX, int64_t n_in, int64_t n_out, int K,
                          int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);
int st_conv_wgrad_planned(int dtype, const void* X, const void* dY, const int32_t* nbr, const int32_t* row_order,
                          const int32_t* tmap, const uint32_t* tmask, void* dW, int64_t n_in, int64_t n_out, int K,
                          int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);

/* st_conv_wgrad_planned in two calls, for a caller that runs the first on another stream beside the feature gradient.
 * On tensor-core shapes st_conv_wgrad_planned first copies dY into the plan's row order (scratch in its workspace), so
 * that the product loads each dY tile as one dense box; the copy depends on dY and row_order alone.
 *   st_conv_wgrad_presort            makes that copy in `workspace`.  ST_ERR_UNSUPPORTED (nothing launched, no error
 *                                    text) when st_conv_wgrad_planned would make none for this layer: call
 *                                    st_conv_wgrad_planned as usual then.
 *   st_conv_wgrad_planned_presorted  the rest, with the same arguments and the same workspace, once the copy is
 *                                    complete on `stream` (an event of the caller's).  Same dW, bit for bit, as
 *                                    st_conv_wgrad_planned.
 * No counterpart in the reference. */
int st_conv_wgrad_presort(int dtype, const void* dY, const int32_t* row_order, int64_t n_out, int K, int cin, int cout,
                          void* workspace, int64_t workspace_bytes, void* stream);
int st_conv_wgrad_planned_presorted(int dtype, const void* X, const void* dY, const int32_t* nbr, const int32_t* row_order,
                                    const int32_t* tmap, const uint32_t* tmask, void* dW, int64_t n_in, int64_t n_out,
                                    int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);

/* The weight gradient walked over the plan of the INVERSE map (from st_map_plan_inverse, or st_map_plan of an
 * inverted map): tiles of 128 INPUT rows, X the per-tile operand, the dY rows of each offset gathered.  Same dW
 * as st_conv_wgrad_planned up to the order of the fp32 additions.  Worth it when the inverse map's rows have the
 * fewer entries (n_in > n_out, a strided layer): its tiles are then the better filled ones.  Tensor-core shapes
 * with 16-byte aligned tensors only (ST_ERR_UNSUPPORTED otherwise).  No counterpart in the reference. */
int64_t st_conv_wgrad_inverse_workspace_bytes(int dtype, int64_t n_in, int K, int cin, int cout);
int st_conv_wgrad_inverse_planned(int dtype, const void* X, const void* dY, const int32_t* row_order, const int32_t* tmap,
                                  const uint32_t* tmask, void* dW, int64_t n_in, int64_t n_out, int K, int cin, int cout,
                                  void* workspace, int64_t workspace_bytes, void* stream);

/* Feature gradient of a submanifold layer over its OWN map (no inverse map, no second plan):
 *   dX[i,:] = sum_k dY[nbr[i,k],:] . W[K-1-k]^T
 * Valid when the map is symmetric, nbr[o,k] = i <=> nbr[i,K-1-k] = o: offsets in opposite pairs and every
 * row returned by the table for its own coordinate (no duplicate or out-of-grid coordinates;
 * st_map_build_symmetric reports that).  Tensor-core shapes only (ST_ERR_UNSUPPORTED otherwise).
 * No counterpart in the reference. */
int st_conv_dgrad_mirrored(int dtype, const void* dY, const void* W, const int32_t* nbr, const int32_t* row_order,
                           const int32_t* tmap, const uint32_t* tmask, void* dX, int64_t n, int K, int cin, int cout,
                           void* workspace, int64_t workspace_bytes, void* stream);

/* Weight gradient without any caller-side memory.  No counterpart in the reference: it exists for
 * hosts that may not allocate device memory around the call -- an inference or training plugin whose
 * memory pool is owned and sized by another runtime, a real-time loop that forbids cudaMalloc after
 * start-up, code running inside a region where allocation would synchronise the device.  The fp32
 * partial sums that st_conv_wgrad() keeps in the caller's workspace are kept here in a fixed array
 * inside the library: st_conv_wgrad_static_max_bytes() bytes (64 MiB) of every GPU that has loaded
 * the library, held until the process exits.  Same arguments and result as st_conv_wgrad(), minus
 * the workspace.  A layer whose partial sums do not fit is refused with ST_ERR_WORKSPACE and a
 * message naming both sizes; nothing is launched in that case.  The call itself allocates nothing
 * and frees nothing.
 *   - The first call on each GPU looks up the device address of the array (with that GPU current);
 *     make that first call outside of any stream capture.  The address is remembered for the life of
 *     the process: it does not survive cudaDeviceReset() or the tear-down of the device's primary
 *     context, after which this entry point must not be called again in the same process.
 *   - All calls on one GPU share the array.  It keeps whatever the last call left in it; each call
 *     overwrites every partial it later reads, so no clearing is needed, but two calls that run on
 *     the GPU at the same time (different streams) would overwrite each other's partials: keep
 *     calls on one GPU ordered. */
int64_t st_conv_wgrad_static_max_bytes(void);
int st_conv_wgrad_static(int dtype, const void* X, const void* dY, const int32_t* nbr, void* dW, int64_t n_in,
                         int64_t n_out, int K, int cin, int cout, void* stream);

/* ---------------------------------------------------------------- normalisation ---------- */

/* Per-sample batch normalisation of sparse features with an optional fused ReLU, as four streaming
 * passes.  Replaces sparse_batch_norm, nn/functional/norm.py:20-112 (statistics per (batch index,
 * channel), biased variance) and the ReLU module that follows it in the reference's networks.
 * `batch` is the int32 batch index of every row (NULL: a single sample); mean, rstd, shift are
 * (B, C) fp32, sums is (B, C, 2) fp32 and is cleared by the call, weight / bias (C) may be NULL.
 *   st_bn_sums            sums[b,c] = ( sum (x - shift), sum (x - shift)^2 ) over the rows of sample b
 *   st_bn_apply           y = relu?((x - mean) * rstd * weight + bias)
 *   st_bn_backward_sums   dz = dy * [relu: output > 0];  sums[b,c] = ( sum dz, sum dz * xhat )
 *   st_bn_backward_apply  dx = rstd * weight * (dz - inv_count[b] * (sums0 + xhat * sums1))
 * A row whose batch index is not in [0, B) takes part in no sum and gets a zero output row; the (B, C)
 * arrays are never touched for it and ST_DEV_BAD_INDEX is OR-ed into *status (device int32, may be NULL). */
int st_bn_sums(int dtype, const void* X, const int32_t* batch, int64_t n, int C, int B, const float* shift, float* sums,
               int32_t* status, void* stream);
int st_bn_apply(int dtype, const void* X, const int32_t* batch, int64_t n, int C, int B, const float* mean,
                const float* rstd, const float* weight, const float* bias, int relu, void* Y, int32_t* status, void* stream);
int st_bn_backward_sums(int dtype, const void* X, const void* dY, const int32_t* batch, int64_t n, int C, int B,
                        const float* mean, const float* rstd, const float* weight, const float* bias, int relu,
                        float* sums, int32_t* status, void* stream);
int st_bn_backward_apply(int dtype, const void* X, const void* dY, const int32_t* batch, int64_t n, int C, int B,
                         const float* mean, const float* rstd, const float* weight, const float* bias, int relu,
                         const float* sums, const float* inv_count, void* dX, int32_t* status, void* stream);

/* ---------------------------------------------------------------- dense conversion ------- */

/* dense (batch, X, Y, Z, C) <- 0, then dense[b, x, y, z, :] = feats[i, :] for every row i with coordinates
 * (b, x, y, z).  The call clears the whole volume itself.  Rows outside the volume (batch >= `batch`, a
 * spatial column outside shape_host) are skipped and ST_DEV_BAD_INDEX is OR-ed into *status (device
 * int32, may be NULL).  Repeated coordinates: one of the rows stays, which one is unspecified (as in the
 * reference, whose stores race).
 * Replaces ToDenseFunction.forward -> _to_dense_fwd_kernel, sparsetriton/utils/to_dense.py:143-203, 30-84. */
int st_to_dense_fwd(int dtype, const void* feats, const void* coords, int coord_dtype, int64_t n, int C, int batch,
                    const int32_t* shape_host, void* dense, int32_t* status, void* stream);

/* grad_feats[i, :] = grad_dense[b, x, y, z, :] (zeros for rows outside the volume).
 * Replaces ToDenseFunction.backward -> _to_dense_bwd_kernel, sparsetriton/utils/to_dense.py:205-240, 87-140. */
int st_to_dense_bwd(int dtype, const void* grad_dense, const void* coords, int coord_dtype, int64_t n, int C, int batch,
                    const int32_t* shape_host, void* grad_feats, void* stream);

/* out[r] = left[r] | right[r]: channel-wise concatenation of two (n, *) feature matrices whose rows are left_bytes and
 * right_bytes long (multiples of 16, 16-byte aligned pointers; else ST_ERR_UNSUPPORTED), and its inverse, which hands
 * the backward pass two contiguous gradients instead of two strided slices.  No reference counterpart (the reference's
 * networks call torch.cat on the features of a skip connection). */
int st_concat_cols(const void* left, const void* right, int64_t n, int left_bytes, int right_bytes, void* out, void* stream);
int st_split_cols(const void* whole, int64_t n, int left_bytes, int right_bytes, void* left, void* right, void* stream);

/* ---------------------------------------------------------------- pooling / upsampling --- */

/* Pooling of a sparse tensor: input voxel `in` belongs to the output cell
 *     out = floor((in + padding - kernel_size/2) / stride)            (per spatial axis; batch kept)
 * and the output rows are the distinct cells in ascending (batch, x, y, z) order, each holding the mean
 * or the maximum of its inputs.  Replaces SparsePoolingFunction, sparsetriton/nn/functional/spatial.py:
 * 26-262 (cells and their order :123-129, reduction kernel :37-88, backward :175-262).  Differences:
 * cells are exact (the reference packs them into 16-bit fields and aliases negative cells), the
 * reduction runs over each row's own segment of a sorted list instead of float atomics (same result
 * from run to run), and the maximum works (the reference's atomic-max form does not compile).
 *
 *   st_pool_count   sort the inputs by cell; *n_out (device or pinned-host int64) <- number of cells.
 *                   Inputs outside [0, shape_host) or with batch >= `batch` join no cell and raise
 *                   ST_DEV_BAD_INDEX in *status.
 *   st_pool_write   (same arguments and workspace, same stream, after _count)
 *                   out_coords (n_out, 4)  the cells, in the coordinate dtype
 *                   in_to_out  (n)         output row of every input (-1: none)
 *                   members    (n)         input rows grouped by output row
 *                   seg_start  (n_out + 1) members[seg_start[o] .. seg_start[o+1]) are the inputs of row o
 *   st_pool_fwd     out[o, :] = mean or max (mode_max != 0) over the members of o, fp32 accumulation
 *   st_pool_bwd     grad_in[i, :] = grad_out[o, :] / count(o)   (mean)
 *                                 = grad_out[o, :] where feats[i, :] == out[o, :], else 0   (max), o = in_to_out[i] */
int64_t st_pool_workspace_bytes(int64_t n);
int st_pool_count(const void* coords, int64_t n, int coord_dtype, int kernel_size, int padding, int stride,
                  const int32_t* shape_host, int batch, void* workspace, int64_t workspace_bytes, int64_t* n_out,
                  int32_t* status, void* stream);
int st_pool_write(const void* coords, int64_t n, int coord_dtype, int kernel_size, int padding, int stride,
                  const int32_t* shape_host, int batch, void* workspace, int64_t workspace_bytes, void* out_coords,
                  int64_t n_out, int32_t* in_to_out, int32_t* members, int32_t* seg_start, void* stream);
int st_pool_fwd(int dtype, const void* feats, int C, const int32_t* members, const int32_t* seg_start, int64_t n_out,
                int mode_max, void* out, void* stream);
int st_pool_bwd(int dtype, const void* grad_out, const void* feats, const void* out, int C, const int32_t* in_to_out,
                const int32_t* seg_start, int64_t n, int mode_max, void* grad_in, void* stream);

/* Nearest-neighbour upsampling: input row i -> output rows i*scale^3 + (dx*scale + dy)*scale + dz with
 * coordinates in*scale + (dx, dy, dz) and the features of row i; backward sums the scale^3 rows in fp32.
 * Replaces SparseUpsampleFunction, sparsetriton/nn/functional/spatial.py:294-505 (kernels :305-396, :446-480). */
int st_upsample_fwd(int dtype, const void* feats, const void* coords, int coord_dtype, int64_t n, int C, int scale,
                    void* out_feats, void* out_coords, void* stream);
int st_upsample_bwd(int dtype, const void* grad_out, int64_t n, int C, int scale, void* grad_in, void* stream);

/* first_row[b] (B int32) <- the smallest row whose batch index is b, -1 when the sample has no row. */
int st_bn_first_rows(const int32_t* batch, int64_t n, int B, int32_t* first_row, void* stream);

/* The statistics of the training forward pass in one call: one pass over X (sums of x - s and (x - s)^2 per
 * (sample, channel), s = the sample's own first row, first_row[b], -1 for an empty sample), then
 *   mean[b,c], rstd[b,c] = 1 / sqrt(biased variance + eps)          (B, C) fp32
 *   running_mean / running_var (C, may be NULL) <- (1 - momentum) * old + momentum * average over the B samples
 * as nn/functional/norm.py:77-94 computes them.  `sums` (B, C, 2) fp32 is scratch; inv_count[b] = 1 / max(rows of b, 1). */
int st_bn_forward_stats(int dtype, const void* X, const int32_t* batch, const int32_t* first_row, int64_t n, int C, int B,
                        const float* inv_count, float eps, float momentum, float* sums, float* mean, float* rstd,
                        float* running_mean, float* running_var, int32_t* status, void* stream);

/* The whole backward pass: st_bn_backward_sums, then dW[c] = sum_b sums[b,c,1], dB[c] = sum_b sums[b,c,0] (either may
 * be NULL) and st_bn_backward_apply (skipped when dX is NULL).  batch_stats = 0: mean / rstd were fixed (inference
 * statistics), the correction terms of dX vanish.  `sums` (B, C, 2) fp32 is scratch. */
int st_bn_backward(int dtype, const void* X, const void* dY, const int32_t* batch, int64_t n, int C, int B, const float* mean,
                   const float* rstd, const float* weight, const float* bias, int relu, int batch_stats,
                   const float* inv_count, float* sums, void* dX, float* dW, float* dB, int32_t* status, void* stream);

/* Hash-on-the-fly forms: no stored map; every tile recomputes
 *   curr = out*lookup_stride - off[k], bounds-checks it against lookup_shape and probes the table.
 * Replace ConvHashOnTheFlyImplicitGEMM forward / backward,
 * funcs/implicit_hashfly_gemm.py:330-452 with kernels :45-148, :151-237, :239-328. */
int64_t st_conv_hashfly_workspace_bytes(int dtype, int64_t n_in, int64_t n_out, int K, int cin, int cout);

int st_conv_fwd_hashfly(int dtype, const void* X, const void* W, const void* out_coords, int coord_dtype,
                        const int32_t* offsets_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                        const int32_t* lookup_shape_host, int lookup_stride, void* Y, int64_t n_in, int64_t n_out,
                        int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream);

/* dX[row(curr),:] += dY[o,:] . W[k]^T, scatter-accumulated in fp32 and then cast to the dtype. */
int st_conv_dgrad_hashfly(int dtype, const void* dY, const void* W, const void* out_coords, int coord_dtype,
                          const int32_t* offsets_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                          const int32_t* lookup_shape_host, int lookup_stride, void* dX, int64_t n_in,
                          int64_t n_out, int K, int cin, int cout, void* workspace, int64_t workspace_bytes,
                          void* stream);

int st_conv_wgrad_hashfly(int dtype, const void* X, const void* dY, const void* out_coords, int coord_dtype,
                          const int32_t* offsets_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                          const int32_t* lookup_shape_host, int lookup_stride, void* dW, int64_t n_in,
                          int64_t n_out, int K, int cin, int cout, void* workspace, int64_t workspace_bytes,
                          void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPARSETRITON_B200_H */
