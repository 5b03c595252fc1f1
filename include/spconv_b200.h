/*
 * spconv_b200 -- C ABI of the B200 (sm_100a) sparse-convolution hot path.
 *
 * One shared library, libspconv_b200.so, replaces the three private modules
 * the reference's operator layer imports at spconv_triton/pytorch/ops.py:24-30
 * (`_impl.pairs`, `_impl.gemm`, `_impl.pool`).  Every entry point below names
 * the reference function it stands in for.
 *
 * Conventions
 *   - all data pointers are DEVICE pointers owned by the caller (PyTorch
 *     allocates them); the library allocates nothing except where noted;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and
 *     the call returns without synchronising, except spc_rulebook_prepare,
 *     which must hand the data-dependent output count back to the host (the
 *     reference synchronises at the same point, _impl/pairs.py:209);
 *   - every function returns an spc_status; spc_last_error() gives the text
 *     of the last failure on the calling thread;
 *   - row-major, contiguous tensors; indices are int32 [n, ndim+1] with the
 *     batch index in column 0, exactly as SparseConvTensor.indices.
 */
#ifndef SPCONV_B200_H_
#define SPCONV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPC_MAX_NDIM 4

typedef enum {
  SPC_OK = 0,
  SPC_ERR_INVALID_ARGUMENT = 1,
  SPC_ERR_CUDA = 2,
  SPC_ERR_WORKSPACE_TOO_SMALL = 3,
  SPC_ERR_HASH_TABLE_FULL = 4,
  SPC_ERR_UNSUPPORTED = 5,
  SPC_ERR_DEVICE_WAIT_EXPIRED = 6,
  SPC_ERR_SIZE_LIMIT = 7,
  SPC_ERR_POINTS_VANISHED = 8
} spc_status;

typedef enum { SPC_F16 = 0, SPC_BF16 = 1, SPC_F32 = 2, SPC_F64 = 3 } spc_dtype;

/* Arithmetic used for fp32 inputs: IEEE fused multiply-add on the CUDA cores,
 * or TF32 on the tensor cores (the reference's live SPCONV_ALLOW_TF32 switch,
 * _impl/gemm.py:460-463).  Ignored for 16-bit inputs, which always multiply
 * exactly and accumulate in fp32. */
typedef enum { SPC_PREC_IEEE = 0, SPC_PREC_TF32 = 1 } spc_precision;

/* Operand preparations for fp32 layers on the tensor cores (spc_tf32_prepare). */
typedef enum { SPC_TF32_ROUND = 0, SPC_TF32_SPLIT_A = 1, SPC_TF32_SPLIT_B = 2 } spc_tf32_mode;

/* Which implementation a GEMM entry point may use.  AUTO picks a tcgen05
 * kernel whenever the shape allows it (gathered rows copied with cp.async;
 * weight slabs loaded by tiled TMA when the channel widths fit a swizzle span,
 * by cp.async otherwise) and the CUDA-core kernel for the rest.  SIMT forces the CUDA-core kernels; TCGEN05 demands a
 * tensor-core kernel (SPC_ERR_UNSUPPORTED if the shape does not fit);
 * TCGEN05_CPASYNC behaves like AUTO but never uses the TMA-fed kernel. */
typedef enum {
  SPC_GEMM_AUTO = 0,
  SPC_GEMM_SIMT = 1,
  SPC_GEMM_TCGEN05 = 2,
  SPC_GEMM_TCGEN05_CPASYNC = 3
} spc_gemm_path;

/* Activation fused into the forward GEMM's store (the reference applies
 * act_type after its kernel, spconv_triton/pytorch/ops.py:63-73). */
typedef enum { SPC_ACT_NONE = 0, SPC_ACT_RELU = 1, SPC_ACT_SIGMOID = 2, SPC_ACT_LEAKY_RELU = 3 } spc_activation;

/* Geometry of one rulebook.  in_shape/out_shape are the spatial shapes before
 * and after the layer (the caller computes out_shape with
 * spc_conv_output_size / spc_deconv_output_size).  For subm the library
 * ignores stride/padding and uses padding = (ksize/2)*dilation, stride 1
 * (_impl/pairs.py:182-187). */
typedef struct {
  int32_t ndim;
  int32_t batch_size;
  int32_t in_shape[SPC_MAX_NDIM];
  int32_t out_shape[SPC_MAX_NDIM];
  int32_t ksize[SPC_MAX_NDIM];
  int32_t stride[SPC_MAX_NDIM];
  int32_t padding[SPC_MAX_NDIM];
  int32_t dilation[SPC_MAX_NDIM];
  int32_t subm;
  int32_t transpose;
} spc_geometry;

/* ---- housekeeping ------------------------------------------------------ */

int spc_version(void);
const char* spc_last_error(void);
/* Number of kernels of this library launched by the process so far (library
 * sorts are not counted).  No counterpart in the reference; used by benchmarks
 * to report how many hand-written kernels a timed region ran. */
long long spc_launch_count(void);
/* Synchronises `stream` and reports whether any kernel of this library gave up
 * on a bounded device-side wait since the last call (SPC_ERR_DEVICE_WAIT_EXPIRED);
 * the flag is cleared.  No counterpart in the reference (its kernels have no
 * device-side waits). */
int spc_check_device_status(void* stream);
/* Queues, on `stream`, a copy of the current device's status word into
 * `pinned_host_word` (page-locked host memory owned by the caller, allocated with
 * cudaHostAlloc / cudaMallocHost so that the device can write it: a one-thread
 * kernel stores the word, no copy engine is involved) and returns without waiting.  The word is non-zero when a kernel gave up on a bounded wait
 * (SPC_ERR_DEVICE_WAIT_EXPIRED) or a rulebook kernel met an index row outside
 * batch_size / spatial_shape (SPC_ERR_INVALID_ARGUMENT).  The host reads the
 * mailbox after work it synchronises on anyway, e.g. at the start of the next
 * forward pass, and then calls spc_check_device_status to clear the word.  No
 * counterpart in the reference (its errors are all raised before launch). */
int spc_post_device_status(int* pinned_host_word, void* stream);

/* ---- output-shape formulas --------------------------------------------- */

/* replaces get_conv_output_size, _impl/pairs.py:59-70 (ksize -1 -> 1). */
int spc_conv_output_size(int ndim, const int32_t* in_shape, const int32_t* ksize,
                         const int32_t* stride, const int32_t* padding,
                         const int32_t* dilation, int32_t* out_shape);
/* replaces get_deconv_output_size, _impl/pairs.py:73-88 (ksize -1 is an error). */
int spc_deconv_output_size(int ndim, const int32_t* in_shape, const int32_t* ksize,
                           const int32_t* stride, const int32_t* padding,
                           const int32_t* dilation, const int32_t* out_padding,
                           int32_t* out_shape);

/* ---- rulebook generation ----------------------------------------------- */

/* Bytes of device scratch the rulebook calls need for this geometry and
 * input count.  The same buffer must be passed, untouched, from
 * spc_rulebook_prepare to the fill call that follows it. */
size_t spc_rulebook_workspace_bytes(const spc_geometry* g, int64_t n_in);

/* Phase 1 of compute_candidates (_impl/pairs.py:126-220): hashes the input
 * coordinates; for strided / transposed layers also enumerates every
 * candidate output coordinate, de-duplicates them in a second hash table,
 * sorts the unique linear coordinates ascending (the order torch.unique
 * gives the reference) and numbers them.  Writes the number of output rows
 * to *n_out_host after synchronising `stream` (subm: n_out = n_in, no
 * synchronisation).  n_out == 0 is the reference's "points vanished" case.
 * The synchronisation spins (cudaStreamSynchronize) unless the environment holds
 * SPC_HOST_WAIT=block when the first call is made: then the thread sleeps on a
 * blocking event, which suits processes with more waiting threads than cores. */
int spc_rulebook_prepare(const spc_geometry* g, const int32_t* indices, int64_t n_in,
                         void* workspace, size_t workspace_bytes, int64_t* n_out_host,
                         void* stream);

/* Phase 2, implicit-gemm format: replaces igemm_pairs, _impl/pairs.py:281-426.
 *   out_indices  [n_out, ndim+1] (NULL for subm: the output rows are the input rows)
 *   pair_fwd     [kv, n_out]  input row feeding (offset, output row), -1 if none
 *   pair_bwd     [kv, n_in]   output row fed by (offset, input row), -1; NULL to skip
 *   mask_fwd     [n_split, n_out, ceil(kv/32)] sorted per-row offset bitmasks
 *   argsort_fwd  [n_split, n_out] original row of each sorted slot
 *   mask_bwd / argsort_bwd  same over the n_in rows of pair_bwd; NULL to skip
 *   split_masks  n_split host words ANDed into mask word 0 (0xFFFFFFFF for
 *                MaskImplicitGemm; the two MaskSplit halves otherwise)
 *   n_out may be smaller than the prepared count (num_out_act_bound): rows
 *   beyond it are dropped, as _impl/pairs.py:318-323 does.
 *   pair_fwd_rowmajor [n_out, kvp] / pair_bwd_rowmajor [n_in, kvp] (kvp = kv
 *   rounded up to 4, padding -1; NULL to skip): the same tables with the kv
 *   entries of a row contiguous.  The GEMM kernels read a tile's entries from
 *   these with a few 16-byte loads per row instead of kv scattered 4-byte
 *   loads; they have no counterpart in the reference. */
int spc_rulebook_igemm(const spc_geometry* g, const int32_t* indices, int64_t n_in,
                       int64_t n_out, void* workspace, size_t workspace_bytes,
                       int32_t* out_indices, int32_t* pair_fwd, int32_t* pair_bwd,
                       int32_t* mask_fwd, int32_t* argsort_fwd, int32_t* mask_bwd,
                       int32_t* argsort_bwd, const uint32_t* split_masks, int n_split,
                       int do_sort, int32_t* pair_fwd_rowmajor, int32_t* pair_bwd_rowmajor,
                       void* stream);

/* The input-side half of spc_rulebook_igemm for strided / transposed layers
 * (pair_bwd, mask_bwd, argsort_bwd, pair_bwd_rowmajor; same meaning), for
 * callers that pass pair_bwd = NULL there and build these tables later or on
 * another stream, off the path of the forward GEMM.  Same part of
 * _impl/pairs.py:281-426 (its pair_bwd / mask_bwd outputs).  Must run after
 * that call has finished with the same workspace (they share scratch). */
int spc_rulebook_igemm_backward(const spc_geometry* g, const int32_t* indices, int64_t n_in,
                                int64_t n_out, void* workspace, size_t workspace_bytes,
                                int32_t* pair_bwd, int32_t* mask_bwd, int32_t* argsort_bwd,
                                const uint32_t* split_masks, int n_split, int do_sort,
                                int32_t* pair_bwd_rowmajor, void* stream);

/* Row-major copy [n, kvp] of a pair table [kv, n] that was not produced by
 * spc_rulebook_igemm (tables converted from the Native format, user tables). */
int spc_pairs_to_rowmajor(const int32_t* pairs, int kv, int64_t n, int32_t* out, void* stream);

/* Phase 2, Native format: replaces native_pairs, _impl/pairs.py:223-278.
 *   pair [2, kv, n_in] (-1 fill): per offset the contributing input rows in
 *   ascending order and their output rows; indice_num_per_loc [kv]. */
int spc_rulebook_native(const spc_geometry* g, const int32_t* indices, int64_t n_in,
                        int64_t n_out, void* workspace, size_t workspace_bytes,
                        int32_t* out_indices, int32_t* pair, int32_t* indice_num_per_loc,
                        void* stream);

/* replaces native_pair_to_tables, _impl/pairs.py:429-469.  pair is
 * [2, kv, n_pair]; pair_fwd [kv, n_out]; pair_bwd [kv, n_in] or NULL. */
int spc_native_to_tables(const int32_t* pair, int kv, int64_t n_pair, int inverse,
                         int32_t* pair_fwd, int64_t n_out, int32_t* pair_bwd, int64_t n_in,
                         void* stream);

/* ---- voxelisation (the step before the rulebook in a LiDAR pipeline) ---- */

/* Replaces PointToVoxel.generate_voxel_with_id, spconv_triton/pytorch/utils.py:72-163.
 *   points [n_points, point_stride] fp32 (first ndim columns are x, y, z..; the
 *   first num_features columns are stored); cmin / vsize / grid_xyz: HOST arrays
 *   of ndim entries in x, y, z order (grid = round((cmax - cmin) / vsize));
 *   voxels [max_voxels, max_points, num_features] fp32 (cleared first when
 *   clear_voxels), indices [max_voxels, ndim] int32 in z, y, x order,
 *   num_per_voxel [max_voxels] int32, pc_voxel_id [n_points] int64 (-1 = out of
 *   range or beyond the voxel cap).  Voxels are numbered by their first point,
 *   points keep arrival order inside a voxel: the result equals the
 *   reference's bit for bit.  *num_voxels_host receives the number of voxels
 *   written (the call synchronises the stream once to read it, where the
 *   reference reads uniq.numel()).  Grids of 2^32 cells or more are rejected. */
size_t spc_voxelize_workspace_bytes(int64_t n_points, int64_t max_voxels);
int spc_voxelize(const float* points, int64_t n_points, int point_stride, int ndim, int num_features,
                 const float* cmin, const float* vsize, const int32_t* grid_xyz, int64_t max_voxels,
                 int max_points, int clear_voxels, int empty_mean, void* workspace,
                 size_t workspace_bytes, float* voxels, int32_t* indices, int32_t* num_per_voxel,
                 int64_t* pc_voxel_id, int64_t* num_voxels_host, void* stream);

/* ---- sparse -> dense (the step after the backbone) ----------------------- */

/* Replaces SparseConvTensor.dense(), spconv_triton/pytorch/core.py:320-334
 * (scatter_nd into zeros, then permute + contiguous for channels_first).
 *   dense: [B, C, *spatial] when channels_first else [B, *spatial, C], elements of
 *   elem_size bytes (2, 4 or 8; the bits are copied); zero-filled, then every
 *   row's channels are written at its coordinate; spatial_shape is a HOST array.
 *   Rows outside the volume are skipped.  spc_dense_gather is the gradient
 *   (features[i, :] = dense[coordinate of row i], 0 for rows outside). */
int spc_dense_scatter(const void* features, const int32_t* indices, int64_t n, int channels, int ndim,
                      int batch_size, const int32_t* spatial_shape, int channels_first, int elem_size,
                      void* dense, void* stream);
int spc_dense_gather(const void* dense, const int32_t* indices, int64_t n, int channels, int ndim,
                     int batch_size, const int32_t* spatial_shape, int channels_first, int elem_size,
                     void* features, void* stream);

/* Dense -> sparse: replaces SparseConvTensor.from_dense, spconv_triton/pytorch/core.py:296-318
 * (torch to_sparse(ndim - 1) there).  dense is channels-last [B, *spatial, C] with `cells` =
 * B * prod(spatial) < 2^31 cells of `channels` elements of elem_size bytes; is_float = 1 treats -0.0
 * as zero.  A cell is kept when any channel is non-zero; rows are numbered in ascending cell order.
 *   spc_from_dense_count    marks and numbers the cells into ws; *count = kept cells (host value;
 *                           synchronises the stream);
 *   spc_from_dense_indices  writes indices [count, ndim + 1] (batch, then coordinates) from the same ws.
 * The features of the rows are then read with spc_dense_gather(channels_first = 0). */
size_t spc_from_dense_workspace_bytes(int64_t cells);
int spc_from_dense_count(const void* dense, int64_t cells, int channels, int elem_size, int is_float,
                         void* ws, size_t ws_bytes, int64_t* count, void* stream);
int spc_from_dense_indices(const void* ws, int64_t cells, int ndim, const int32_t* spatial_shape,
                           int32_t* indices, void* stream);

/* Global pooling: replaces SparseGlobalMaxOrAvgPool.forward, spconv_triton/pytorch/pool.py:238-265
 * (with global_pool_rearrange, ops.py:436-450).  features [n, channels] of dtype (fp16, bf16, fp32),
 * indices [n, idx_width] int32 with the sample number in column 0 (rows of other samples than
 * 0..batch-1 are ignored; any row order).
 *   is_mean = 0: out [batch, channels] = per-sample maximum (NaN propagates), argmax [batch, channels]
 *                (or NULL) = the smallest row that holds it, -1 for a sample without rows;
 *   is_mean = 1: out [batch] = per-sample mean of CHANNEL 0 (what upstream returns, pool.py:258-261),
 *                accumulated in fp64; NaN for a sample without rows.
 * counts [batch] int32 (or NULL) receives the rows per sample. */
size_t spc_global_pool_workspace_bytes(int batch, int channels);
int spc_global_pool(const void* features, const int32_t* indices, int64_t n, int channels, int idx_width,
                    int batch, int dtype, int is_mean, void* ws, size_t ws_bytes, void* out,
                    int32_t* argmax, int32_t* counts, void* stream);

/* ---- key -> value hash table and misaligned sparse add ------------------- */

/* A fixed-capacity GPU hash table; replaces HashTable, spconv_triton/pytorch/hash.py:15-110
 * (sorted arrays + searchsorted there).  The table lives in ONE caller-owned device buffer of
 * spc_hash_bytes(capacity) bytes; capacity = number of slots, a power of two (the host wrapper
 * takes the power of two >= 2 * max_size).  Keys are int32 or int64 (key_bytes 4 / 8; INT64_MIN
 * is reserved), values are the bits of any 1/2/4/8-byte type.
 *   spc_hash_clear     empties the table.
 *   spc_hash_insert    hash.py:38-60: stores keys[i] -> values[i] (0 when values is NULL); of equal
 *                      keys in one call the LAST wins.  `epoch` must grow with every insert call on a
 *                      table (it orders the writers; 24 bits).
 *   spc_hash_counters  host read (synchronises the stream): number of stored keys and of keys an
 *                      insert dropped because the table was full ("hash table full", hash.py:59-60).
 *   spc_hash_query     hash.py:62-79: out_values[i] = value or 0, is_empty[i] = 1 when absent.
 *   spc_hash_update    insert_exist_keys, hash.py:81-92: overwrites values of stored keys only.
 *   spc_hash_items     hash.py:94-110: the `count` stored pairs in ascending key order into
 *                      out_keys / out_values (either may be NULL; at most out_limit entries written).
 *                      assign_kind -1 keeps the values; 0 / 1 / 2 first replaces them by the rank
 *                      in that order as integer / float / double (assign_arange_, hash.py:94-99).
 *                      `count` = the stored-key count read with spc_hash_counters.  key_bits: when
 *                      every key is in [0, 2^key_bits) the sort stops there; 0 = all 64 bits. */
size_t spc_hash_bytes(int64_t capacity);
int spc_hash_clear(void* table, int64_t capacity, void* stream);
int spc_hash_insert(void* table, int64_t capacity, const void* keys, int key_bytes, const void* values,
                    int val_bytes, int64_t n, uint64_t epoch, void* stream);
int spc_hash_counters(const void* table, int64_t capacity, int64_t* stored, int64_t* dropped, void* stream);
int spc_hash_query(const void* table, int64_t capacity, const void* keys, int key_bytes, int64_t n,
                   void* out_values, int val_bytes, uint8_t* is_empty, void* stream);
int spc_hash_update(void* table, int64_t capacity, const void* keys, int key_bytes, const void* values,
                    int val_bytes, int64_t n, uint8_t* found, void* stream);
size_t spc_hash_items_workspace_bytes(int64_t count);
int spc_hash_items(void* table, int64_t capacity, int64_t count, int assign_kind, int key_bits, void* ws,
                   size_t ws_bytes, void* out_keys, int key_bytes, void* out_values, int val_bytes,
                   int64_t out_limit, void* stream);

/* _indice_to_scalar, spconv_triton/pytorch/functional.py:415-426: keys[i] = the row-major linear
 * coordinate of indices[i, 0..width) over shape[0..width) (HOST array: batch size, then the spatial
 * shape), as int32 or int64 (key_bytes 4 / 8). */
int spc_coords_to_keys(const int32_t* indices, int64_t n, int width, const int64_t* shape, int key_bytes,
                       void* keys, void* stream);

/* The accumulation of sparse_add_hash_based, spconv_triton/pytorch/functional.py:476-480:
 *   dst[rows[i], :] += src[i, :]  and  idx_dst[rows[i], :] = idx_src[i, :]  (idx_src may be NULL)
 * for rows that are distinct within the call (no atomics); rows outside [0, dst_rows) are skipped.
 * src [n, channels] and dst [dst_rows, channels] of `dtype` (spc_dtype).  spc_rows_gather is its
 * gradient: dst[i, :] = src[rows[i], :]. */
int spc_rows_scatter_add(const void* src, const int32_t* rows, int64_t n, int channels, int dtype,
                         int64_t dst_rows, void* dst, const int32_t* idx_src, int idx_width,
                         int32_t* idx_dst, void* stream);
int spc_rows_gather(const void* src, const int32_t* rows, int64_t n, int channels, int dtype,
                    int64_t src_rows, void* dst, void* stream);

/* ---- implicit gather-GEMM ---------------------------------------------- */

/* Forward: replaces conv_forward, _impl/gemm.py:501-568.
 *   out[m, n] = sum_k sum_c features[pair_fwd[k, m], c] * weight[n, k, c] (+ bias[n])
 *   features [n_in, c_in] dtype; weight [c_out, kv, c_in] dtype (KRSC);
 *   bias [c_out] dtype or NULL; out [n_out, c_out] out_dtype;
 *   mask_argsort [n_out] or NULL: the order in which rows are grouped into
 *   tiles (rows with equal offset bitmasks become neighbours);
 *   pair_fwd_rowmajor [n_out, kvp] or NULL: the row-major copy of pair_fwd
 *   (spc_rulebook_igemm / spc_pairs_to_rowmajor); optional, only faster;
 *   out_scale, out_shift: fp32 [c_out] or both NULL; when given the store is
 *   out = act((acc + bias) * out_scale + out_shift), i.e. an inference
 *   BatchNorm folded into the layer; act / act_alpha: spc_activation and the
 *   LeakyReLU slope. */
int spc_conv_forward(const void* features, const void* weight, const void* bias,
                     const int32_t* pair_fwd, const int32_t* pair_fwd_rowmajor,
                     const int32_t* mask_argsort, void* out,
                     int64_t n_in, int64_t n_out, int c_in, int c_out, int kv, int dtype,
                     int out_dtype, int precision, int path, const float* out_scale,
                     const float* out_shift, int act, float act_alpha, void* stream);

/* 1 if spc_conv_forward for this layer reads the column-major table pair_fwd, 0 if the
 * row-major copy is all it reads (the tcgen05 kernel with TMA-fed weights).  In the
 * second case pair_fwd may be NULL as long as pair_fwd_rowmajor is given, which lets a
 * caller that owns both tables not write the one nobody reads (spc_sequence_forward
 * does).  No counterpart in the reference, whose kernels read one table layout
 * (spconv_triton/pytorch/ops.py:259-305). */
int spc_conv_forward_needs_colmajor(int c_in, int c_out, int kv, int dtype, int out_dtype, int precision,
                                    int path);

/* spc_conv_forward with a residual connection fused into the store:
 *   out[m, n] = act((acc + bias[n]) * scale[n] + shift[n]) + residual[m, n]
 * residual [n_out, c_out] has the OUTPUT dtype (16-byte aligned, NULL = none) and is
 * added in fp32 before the single rounding of the store.  Replaces the separate
 * pass the reference makes for `add_input` after its kernel
 * (spconv_triton/pytorch/conv.py:503-511). */
int spc_conv_forward_residual(const void* features, const void* weight, const void* bias,
                              const int32_t* pair_fwd, const int32_t* pair_fwd_rowmajor,
                              const int32_t* mask_argsort, void* out, int64_t n_in, int64_t n_out,
                              int c_in, int c_out, int kv, int dtype, int out_dtype, int precision,
                              int path, const float* out_scale, const float* out_shift, int act,
                              float act_alpha, const void* residual, void* stream);

/* Input gradient: replaces conv_backward_input, _impl/gemm.py:571-631.
 *   din[j, c] = sum_k sum_n grad_out[pair_bwd[k, j], n] * weight[n, k, c]
 *   grad_out [n_out, c_out]; din [n_in, c_in], both `dtype`. */
int spc_conv_backward_input(const void* grad_out, const void* weight,
                            const int32_t* pair_bwd, const int32_t* pair_bwd_rowmajor,
                            const int32_t* mask_argsort, void* din,
                            int64_t n_in, int64_t n_out, int c_in, int c_out, int kv,
                            int dtype, int precision, int path, void* stream);

/* fp32 layers on the tensor cores.  The TF32 tensor-core path uses the upper 19
 * bits of each fp32 operand.  spc_tf32_prepare writes a prepared copy of a
 * row-major fp32 matrix [rows, cols]:
 *   SPC_TF32_ROUND    dst [rows, cols]     every value rounded to the nearest TF32
 *                     number, the rounding the reference's tl.dot applies when
 *                     SPCONV_ALLOW_TF32 is set (_impl/gemm.py:55-62);
 *   SPC_TF32_SPLIT_A  dst [rows, 3 cols]   rows [hi | lo | hi], x = hi + lo;
 *   SPC_TF32_SPLIT_B  dst [rows, 3 cols]   rows [hi | hi | lo].
 * A convolution whose gathered operand was split with SPLIT_A and whose weight
 * with SPLIT_B (reduction length 3 c_in, precision SPC_PREC_TF32) computes
 * hi hi + lo hi + hi lo, i.e. the fp32 product to 2^-22: this is how IEEE-mode
 * fp32 layers (the reference's default, _impl/gemm.py:11-13) run on tcgen05.
 * spc_tf32_prepare_weight does the same for a KRSC weight [c_out, kv, c_in] ->
 * [c_out, kv, m c_in], or with `transpose` -> [c_in, kv, m c_out] (the operand
 * of the input gradient written as a forward convolution of grad_out), m = 1
 * (ROUND) or 3 (SPLIT_*).  No counterpart in the reference. */
int spc_tf32_prepare(const float* src, float* dst, int64_t rows, int cols, int mode, void* stream);
int spc_tf32_prepare_weight(const float* weight, float* dst, int c_out, int kv, int c_in,
                            int transpose, int mode, void* stream);

/* Bytes of device scratch spc_conv_backward_weight needs (fp32 partial sums
 * of the split reduction). */
size_t spc_conv_backward_weight_workspace_bytes(int64_t n_out, int c_in, int c_out, int kv);

/* Weight gradient: replaces conv_backward_weight, _impl/gemm.py:634-713.
 *   dweight[n, k, c] = sum over m with pair_fwd[k, m] >= 0 of
 *                      features[pair_fwd[k, m], c] * grad_out[m, n]
 *   dweight [c_out, kv, c_in] dtype.  The reduction over rows is split into
 *   chunks whose fp32 partial sums live in `workspace` and are added in a
 *   fixed order, so the result is deterministic. */
int spc_conv_backward_weight(const void* features, const void* grad_out,
                             const int32_t* pair_fwd, void* dweight, void* workspace,
                             size_t workspace_bytes, int64_t n_in, int64_t n_out, int c_in,
                             int c_out, int kv, int dtype, int precision, int path,
                             void* stream);

/* Weight gradient for callers that cannot provide a workspace and must not
 * allocate: the same sum as spc_conv_backward_weight, but the fp32 partial sums
 * of the split reduction live in a 16 MiB array built into the library (held
 * by every GPU that loads it, until the process exits).  It has no counterpart
 * in the reference.
 *   - it always runs the CUDA-core kernel, so its result is bit-identical to
 *     spc_conv_backward_weight called with path = SPC_GEMM_SIMT, and equal only
 *     within rounding to the default path, which uses the tensor cores (another
 *     split and summation order) for 16-bit shapes; for those shapes it is also
 *     roughly ten times slower than the default path;
 *   - shapes whose partial sums exceed spc_conv_backward_weight_noalloc_max_bytes()
 *     are rejected with SPC_ERR_SIZE_LIMIT (compare with
 *     spc_conv_backward_weight_workspace_bytes() for the same arguments);
 *   - the first call on a device looks up the array's device address; make that
 *     call before any stream capture on the device;
 *   - all calls on a device share the array: calls that overlap on the GPU race,
 *     so issue them on one stream or order them yourself;
 *   - neither this call nor anything it launches allocates or frees memory. */
size_t spc_conv_backward_weight_noalloc_max_bytes(void);
int spc_conv_backward_weight_noalloc(const void* features, const void* grad_out,
                                     const int32_t* pair_fwd, void* dweight, int64_t n_in,
                                     int64_t n_out, int c_in, int c_out, int kv, int dtype,
                                     void* stream);

/* ---- sparse pooling ---------------------------------------------------- */

/* replaces maxpool_forward, _impl/pool.py:260-288: accumulator starts at 0. */
int spc_maxpool_forward(const void* features, const int32_t* pair_fwd, void* out,
                        int64_t n_out, int channels, int kv, int dtype, void* stream);
/* replaces maxpool_backward, _impl/pool.py:291-330: every input equal to the
 * output receives the gradient. */
int spc_maxpool_backward(const void* features, const void* out_features, const void* grad_out,
                         const int32_t* pair_bwd, void* din, int64_t n_in, int channels,
                         int kv, int dtype, void* stream);
/* replaces avgpool_forward, _impl/pool.py:333-364: mean over the inputs that
 * are present; count [n_out] int32 (may be NULL). */
int spc_avgpool_forward(const void* features, const int32_t* pair_fwd, void* out,
                        int32_t* count, int64_t n_out, int channels, int kv, int dtype,
                        void* stream);
/* replaces avgpool_backward, _impl/pool.py:367-397: the gradient is
 * multiplied by the window count (the reference's behaviour). */
int spc_avgpool_backward(const void* grad_out, const int32_t* pair_bwd, const int32_t* count,
                         void* din, int64_t n_in, int channels, int kv, int dtype,
                         void* stream);

/* ---- a chain of convolutions in one call --------------------------------- */

/* One layer of spc_sequence_forward: a sparse convolution with kernel volume <= 32
 * (the implicit-gemm algorithm), optionally followed by a folded inference
 * BatchNorm (scale / shift) and an activation, as spc_conv_forward applies them.
 * `rulebook` is the index of the layer whose rulebook this layer uses: its own
 * index if it generates one; the index of an earlier SUBMANIFOLD layer of the
 * same level to share that one (the reference's indice_key reuse,
 * spconv_triton/pytorch/conv.py:211-219). */
typedef struct {
  spc_geometry geom;
  int32_t rulebook;
  int32_t c_in, c_out;
  const void* weight;   /* [c_out, kv, c_in], dtype of the features */
  const void* bias;     /* [c_out] or NULL */
  const float* scale;   /* [c_out] fp32 or NULL (with shift) */
  const float* shift;
  int32_t act;          /* spc_activation */
  float act_alpha;
} spc_seq_layer;

/* What a layer produced: row counts and byte offsets into the arena
 * (UINT64_MAX = not produced: a layer that shares a rulebook has only
 * `features`; submanifold layers have no out_indices). */
typedef struct {
  int64_t n_in, n_out;
  uint64_t workspace, workspace_bytes;   /* rulebook workspace, as spc_rulebook_prepare left it */
  uint64_t out_indices;                  /* [n_out, ndim+1] int32 */
  uint64_t pair_fwd;                     /* [kv, n_out] int32; not produced when no layer that uses the
                                            rulebook reads it (spc_conv_forward_needs_colmajor): it is
                                            the transpose of pair_fwd_rowmajor[:, :kv] */
  uint64_t pair_fwd_rowmajor;            /* [n_out, kvp] int32 */
  uint64_t pair_mask;                    /* [n_out] int32 (one split, one word) */
  uint64_t mask_argsort;                 /* [n_out] int32 */
  uint64_t num_per_loc;                  /* [kv] int32, zeros (as igemm_pairs returns) */
  uint64_t features;                     /* [n_out, c_out], dtype */
  int64_t masks_are_exact;               /* 1: pair_mask / mask_argsort are what spc_rulebook_igemm emits (the
                                            mask words sorted ascending, stable, and their argsort); 0: the pass
                                            ordered the rows for its own GEMMs by a key that packs rows with
                                            common kernel offsets into the same 128-row tile: mask_argsort is
                                            that order, pair_mask the sorted keys, and the exact pair is the
                                            stable sort of the mask words of pair_fwd_rowmajor (bit k of a
                                            row's word = entry k >= 0) */
} spc_seq_result;

/* Inference forward of `n_layers` convolutions applied one after the other to
 * (indices [n_in, ndim+1], features [n_in, layers[0].c_in]); replaces the
 * layer-by-layer loop of SparseSequential.forward
 * (spconv_triton/pytorch/modules.py:30-100) over ops.get_indice_pairs_implicit_gemm
 * and ops.implicit_gemm for such a chain.  Every output, table and workspace is
 * placed in `arena` (256-byte aligned device memory owned by the caller, which
 * must stay alive while the results are used); `results[i]` says where.
 * Rulebooks of strided layers are generated on `stream_chain`, those of
 * submanifold layers on `stream_side`, the GEMMs on `stream_main`, ordered by
 * events; on return `stream_main` has been made to wait for both other streams.
 * The call blocks on `stream_chain` once per strided layer (the read of its
 * output count, as _impl/pairs.py:209 does).
 * Returns SPC_ERR_WORKSPACE_TOO_SMALL with *arena_needed set to a larger size to
 * retry with when the arena is too small (nothing useful has been produced
 * then), SPC_ERR_POINTS_VANISHED when a layer has no output rows.
 * 16-bit features only; the input-side tables of strided layers are not built
 * (spc_rulebook_igemm_backward builds them from results[i].workspace). */
int spc_sequence_forward(const spc_seq_layer* layers, int n_layers, const int32_t* indices,
                         const void* features, int64_t n_in, int dtype, void* arena,
                         size_t arena_bytes, size_t* arena_needed, spc_seq_result* results,
                         void* stream_main, void* stream_chain, void* stream_side);

#ifdef __cplusplus
}
#endif
#endif /* SPCONV_B200_H_ */
