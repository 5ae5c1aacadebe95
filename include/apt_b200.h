/*
 * apt_b200.h — C ABI of libapt_b200.so: the mini-batch data path of APT
 * (neighbour sampling, relabelling, cache-aware feature gather, seed/feature
 * shuffle between GPUs, SpMM/SDDMM over sampled blocks) as hand-written
 * sm_100a CUDA.
 *
 * Conventions
 *  - Every pointer is a raw device pointer unless its comment says "host".
 *    "uva" pointers are page-locked host allocations that the device can
 *    dereference (cudaHostRegister / cudaHostAlloc).
 *  - Ids and offsets are int64_t, like the reference's IdType (src/utils.h:14).
 *  - `stream` is a cudaStream_t passed as void*. Calls are stream-ordered and
 *    never synchronise the host unless the comment says so.
 *  - Sizes are host integers. Where an entry point also takes a `*_dev`
 *    pointer, that device word (if not NULL) overrides the host size at run
 *    time, the host size then being only an upper bound that sized grids and
 *    buffers: a chain of operators can so run without the host ever reading
 *    an intermediate count.
 *  - Outputs and workspaces are allocated by the caller. No entry point in
 *    this header allocates device memory except apt_p2p_create.
 *  - Return value: APT_OK or an apt_status; apt_last_error() gives the text.
 *    Nothing here aborts the process, traps the GPU or waits without a bound.
 *  - Each entry point cites the reference function (file:line inside the
 *    kaihaoma/APT tree) whose role it takes.
 */
#ifndef APT_B200_H_
#define APT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum apt_status {
  APT_OK = 0,
  APT_ERR_BAD_ARG = 1,   /* null pointer, negative size, unsupported dtype/alignment */
  APT_ERR_CUDA = 2,      /* a CUDA runtime call failed */
  APT_ERR_TIMEOUT = 3,   /* a bounded wait on a peer ran out */
  APT_ERR_OOB = 4,       /* an id outside the registered tables was seen */
  APT_ERR_CAPACITY = 5   /* workspace / inbox too small for this call */
} apt_status;

/* Element types of feature rows. The gather and shuffle are byte copies and
 * only need the element size; SpMM/SDDMM compute in fp32 and round once. */
typedef enum apt_dtype { APT_F32 = 0, APT_BF16 = 1, APT_F16 = 2 } apt_dtype;

/* Bits of the device-side status word (int32) several kernels OR into. */
#define APT_FLAG_ID_OUT_OF_RANGE 1  /* node id < 0 or >= num_nodes */
#define APT_FLAG_FEAT_NOT_EXIST  2  /* feat_pos_map == -1: row neither cached nor on host */
#define APT_FLAG_ZERO_DEGREE     4  /* sampled a node with no in-neighbour */
#define APT_FLAG_TABLE_FULL      8  /* relabel hash table overflow (workspace too small) */
#define APT_FLAG_PEER_TIMEOUT    16 /* a peer's flag did not arrive in time */
#define APT_FLAG_NOT_GROUPED     32 /* a block operator got edges not grouped by destination */
#define APT_FLAG_SIZE_MISMATCH   64 /* a peer sent another number of rows than the reduction expects */

const char* apt_last_error(void);
int apt_version(void);

/* Number of kernels this library has launched in this process, and a reset.
 * The benchmark reports it as its launch count. */
int64_t apt_launch_count(void);
void apt_launch_count_reset(void);

/* One stream-ordered copy of nbytes between any two of device memory and
 * page-locked host memory (the direction follows from the pointers). It is
 * what the samplers put into a captured CUDA graph to bring the call-id base
 * in and the block of device-side counts out: a captured copy reads its host
 * source when the replay runs. No counterpart in the reference, which reads
 * its sizes with blocking copies (src/sampling.cc:176-185). */
int apt_memcpy_async(void* dst, const void* src, size_t nbytes, void* stream);

/* Optional per-kernel timing. When enabled, every launch of a tagged kernel
 * is bracketed by CUDA events on its own stream; apt_profile_read
 * synchronises those events and returns the summed milliseconds and launch
 * count of one tag ("gather_hit", "gather_miss", "sample", "relabel", ...)
 * then forgets them. Off by default (no events are recorded). */
int apt_profile_enable(int on);
int apt_profile_read(const char* tag, double* total_ms, int64_t* launches);

/* Tuning knobs for measurements; the defaults are what the benchmark uses.
 *   gather_miss_mode   0 16-byte ld.global.nc loads (default),
 *                      1 bulk copies (cp.async.bulk) staged through shared memory
 *   gather_miss_blocks blocks of the miss-copy kernel (default 148)
 *   gather_miss_kb_per_block  0 (default): every block of the miss copy takes part; k > 0: one block per
 *                      k KiB to fetch (at least 16), the rest leave at once and keep their SM slots free.
 *                      The samplers set 128 for the launches they capture on a lane, where other
 *                      mini-batches' kernels run beside the copy.
 *   gather_hit_mode    copy of the cache hits: 0 one resident wave, two groups of rows in flight per warp,
 *                      1 bulk copies (cp.async.bulk) staged through shared memory,
 *                      2 grid-stride blocks, one group of rows per warp at a time
 *   gather_hit_waves   mode 2: cap on the grid, in units of 148 x 8 blocks (default 4)
 *   relabel_small      1 (default): layers of up to 8192 items are relabelled by one block with
 *                      the hash table in shared memory; 0: always the multi-block path */
int apt_set_tunable(const char* name, int64_t value);

/* ------------------------------------------------------------------ sampling
 * Uniform fanout sampling of in-neighbours from a CSC graph, one dense row of
 * `fanout` ids per seed. Takes the role of LocalSampleNeighbors /
 * _CSRRowWiseSampleReplaceKernel (src/cuda/npc_kernel.cu:248-316) behind
 * LocalSamplingNeibhorsOneLayer (src/sampling.cc:13-17).
 *
 *   p = adj_pos_map[v];  p >= 0 : row p of (dev_indptr, dev_indices)
 *                        p <  0 : row -(p)-2 of (uva_indptr, uva_indices)
 *   replace != 0:  out[j*fanout+i] = indices[start + draw(j,i) % deg]
 *   replace == 0:  Floyd selection of `fanout` distinct edge slots when
 *                  deg > fanout (fanout <= 32); otherwise every neighbour once,
 *                  then draws with replacement for the remaining slots.
 *   deg == 0:      the row is filled with v itself and APT_FLAG_ZERO_DEGREE is
 *                  set (the reference leaves the row uninitialised).
 *   draw(j,i) = word (i & 3) of Philox4x32-10 with key (key_lo, key_hi) and
 *               counter (j & 0xffffffff, j >> 32, i >> 2, call_id).
 * adj_pos_map may be NULL: every node then reads (uva_indptr, uva_indices),
 * which may be plain device memory holding the whole graph.
 * call_id_base_dev (may be NULL) is a device word added to call_id at run time,
 * so that a captured CUDA graph draws a fresh stream at every replay.
 */
int apt_sample_csc_fanout(const int64_t* seeds, int64_t num_seeds,
                          const int64_t* num_seeds_dev, int fanout,
                          const int64_t* adj_pos_map, int64_t num_nodes,
                          const int64_t* dev_indptr, const int64_t* dev_indices,
                          const int64_t* uva_indptr, const int64_t* uva_indices,
                          uint64_t key, uint32_t call_id,
                          const int64_t* call_id_base_dev, int replace,
                          int64_t* out_neighbors, int32_t* status_word,
                          void* stream);

/* ------------------------------------------------------------------ relabel
 * First-occurrence unique of cat(seeds, neighbors) and the position of every
 * neighbour in it. Takes the role of TensorRelabelCSC (src/cuda/relabel.cu:
 * 175-185; Unique :78-151, Relabel :153-173) behind RelabelCSC
 * (src/relabel.cc:9-15).
 *
 *   out_unique     int64[num_seeds + num_neighbors] (only the first U written)
 *   out_relabeled  int64[num_neighbors]
 *   out_num_unique int64[1] device word receiving U
 * workspace: apt_relabel_workspace_bytes(num_seeds + num_neighbors) bytes or
 * more, 256-byte aligned, emptied ONCE with apt_relabel_workspace_init after
 * allocation; every call leaves it empty again (it releases the table slots it
 * used), so no clearing pass runs per call. Always pass the same size for the
 * same workspace: the layout is derived from it.
 * With num_seeds_dev the real seed count S comes from the device and the
 * neighbours are taken to be S * (num_neighbors / num_seeds) (a fixed fanout).
 * A negative id is not an id (-1 is what an operator upstream leaves for an id it
 * could not resolve): it is left out of out_unique, relabelled to -1, and
 * APT_FLAG_ID_OUT_OF_RANGE is set. (The reference would take -1 for its
 * empty-slot mark, src/cuda/relabel.cu:70.)
 */
size_t apt_relabel_workspace_bytes(int64_t num_items);
int apt_relabel_workspace_init(void* workspace, size_t workspace_bytes, void* stream);
int apt_relabel_csc(const int64_t* seeds, int64_t num_seeds,
                    const int64_t* num_seeds_dev,
                    const int64_t* neighbors, int64_t num_neighbors,
                    void* workspace, size_t workspace_bytes,
                    int64_t* out_unique, int64_t* out_relabeled,
                    int64_t* out_num_unique, int32_t* status_word,
                    void* stream);

/* Sampling and relabelling of one layer in one call: what
 * LocalSamplingNeibhorsOneLayer followed by RelabelCSC compute (src/sampling.cc:13-17,
 * src/relabel.cc:9-15; python/npc/sampler.py:117-121 calls them back to back),
 * with the draws of apt_sample_csc_fanout (replace != 0) and the outputs of
 * apt_relabel_csc on those neighbours. The sampling kernel enters every id into
 * the relabel table while it holds it, so the neighbour list is not read back;
 * out_neighbors (int64[num_seeds * fanout]) may be NULL when the caller only needs
 * the block. Layers of up to 8192 items are one launch. Workspace as for
 * apt_relabel_csc with num_seeds * (1 + fanout) items. */
int apt_sample_relabel_csc(const int64_t* seeds, int64_t num_seeds,
                           const int64_t* num_seeds_dev, int fanout,
                           const int64_t* adj_pos_map, int64_t num_nodes,
                           const int64_t* dev_indptr, const int64_t* dev_indices,
                           const int64_t* uva_indptr, const int64_t* uva_indices,
                           uint64_t key, uint32_t call_id,
                           const int64_t* call_id_base_dev,
                           void* workspace, size_t workspace_bytes,
                           int64_t* out_neighbors, int64_t* out_unique,
                           int64_t* out_relabeled, int64_t* out_num_unique,
                           int32_t* status_word, void* stream);

/* ----------------------------------------------------------- owner bucketing
 * Stable partition of ids by owning rank. Takes the role of ClusterAndPermute
 * (src/cuda/npc_kernel.cu:318-382, :434-470) inside ShuffleSeeds
 * (src/sampling.cc:159-193).
 *
 *   owner(v): d = shuffle_id_offset; while d+1 < world_size and
 *             min_vids[d+1] <= v: ++d;  if d outside [node_beg,node_end): d = rank
 *   out_sorted[ out_perm[i] ] = ids[i]; ids of one owner keep their input order
 *   out_bucket_sizes int64[world_size + 1] (sizes, then their total);
 *   out_bucket_offsets int64[world_size] = inclusive cumsum.
 * min_vids is a device array of world_size+1 entries; world_size <= 32.
 * workspace: apt_bucket_workspace_bytes(num_ids, world_size) bytes.
 */
size_t apt_bucket_workspace_bytes(int64_t num_ids, int world_size);
int apt_bucket_by_owner(const int64_t* ids, int64_t num_ids,
                        const int64_t* num_ids_dev,
                        const int64_t* min_vids, int world_size,
                        int64_t shuffle_id_offset, int rank, int node_beg,
                        int node_end, void* workspace, size_t workspace_bytes,
                        int64_t* out_sorted, int64_t* out_perm,
                        int64_t* out_bucket_sizes, int64_t* out_bucket_offsets,
                        void* stream);

/* ------------------------------------------------------- sorted unique + inverse
 * Ascending unique of ids within [id_lo, id_hi) and, per input, its position
 * in that unique list. Takes the role of torch::_unique2(sorted, inverse) in
 * NPSampleAndShuffle (src/sampling.cc:58-59). A two-level bitmap over the id
 * range replaces the sort. Ids outside the range set APT_FLAG_ID_OUT_OF_RANGE
 * and get inverse -1.
 *   out_unique int64[min(num_ids, id_hi-id_lo)], out_inverse int64[num_ids],
 *   out_num_unique int64[1] device word.
 * workspace: apt_unique_workspace_bytes(id_hi - id_lo) bytes, zeroed with
 * apt_unique_workspace_init after allocation and again whenever it is used with
 * another range width (the layout follows the width); every call leaves it
 * zeroed again (it clears the bits it set), so a call costs O(num_ids + range/1024).
 */
size_t apt_unique_workspace_bytes(int64_t id_range);
int apt_unique_workspace_init(void* workspace, size_t workspace_bytes, void* stream);
int apt_unique_sorted(const int64_t* ids, int64_t num_ids,
                      const int64_t* num_ids_dev, int64_t id_lo, int64_t id_hi, void* workspace, size_t workspace_bytes,
                      int64_t* out_unique, int64_t* out_inverse,
                      int64_t* out_num_unique, int32_t* status_word,
                      void* stream);

/* ---------------------------------------------------------------- gather
 * Cache-aware feature-row gather. Takes the role of IndexSelectAll /
 * _CSRRowWiseLoadSubtensorAlignedAllKernel (src/cuda/npc_kernel.cu:187-246)
 * behind LoadSubtensor (src/load_subtensor.cc:19-40).
 *
 *   p = feat_pos_map[index[r]]
 *   p >= 0 : out[r] = dev_feats row p            (dev_row_bytes each)
 *   p < -1 : out[r] = uva_feats row -(p)-2, bytes [uva_col_offset_bytes,
 *            uva_col_offset_bytes + dev_row_bytes) of a uva_row_bytes row
 *   p == -1: out[r] = 0 and APT_FLAG_FEAT_NOT_EXIST (the reference reads out
 *            of bounds here)
 * Rows are opaque bytes, so fp32/bf16/fp16 tables share the code.
 * Three kernels on `stream`: classify (decode p, compact the miss list), the
 * hit copy out of the HBM cache and the miss copy over the host link.
 * workspace: apt_gather_workspace_bytes(num_rows) bytes; needs no initialisation.
 * apt_gather_rows_from only produces output rows [*first_row_dev, num_rows) (a
 * device word; NULL: 0): a caller that already holds the leading rows, e.g. the
 * destination nodes of a block whose rows it fetched while the block was still
 * being built, gathers the rest with the same index and output arrays.
 */
size_t apt_gather_workspace_bytes(int64_t num_rows);
int apt_gather_rows_from(const int64_t* index, int64_t num_rows,
                         const int64_t* num_rows_dev, const int64_t* first_row_dev,
                         const int64_t* feat_pos_map, int64_t num_nodes,
                         const void* dev_feats, int64_t num_dev_rows,
                         int64_t dev_row_bytes, const void* uva_feats,
                         int64_t num_uva_rows, int64_t uva_row_bytes,
                         int64_t uva_col_offset_bytes, void* out, void* workspace,
                         size_t workspace_bytes, int32_t* status_word, void* stream);
int apt_gather_rows(const int64_t* index, int64_t num_rows,
                    const int64_t* num_rows_dev,
                    const int64_t* feat_pos_map, int64_t num_nodes,
                    const void* dev_feats, int64_t num_dev_rows,
                    int64_t dev_row_bytes, const void* uva_feats,
                    int64_t num_uva_rows, int64_t uva_row_bytes,
                    int64_t uva_col_offset_bytes, void* out, void* workspace,
                    size_t workspace_bytes, int32_t* status_word, void* stream);

/* Gather for callers that cannot allocate device memory. No counterpart in the
 * reference, whose gather allocates its output and keeps no scratch.
 *
 * Who needs it: code that runs where cudaMalloc is not an option — inside a
 * memory pool whose owner has handed out every byte already (an inference
 * server that pre-plans all device memory at start-up), in a callback or a
 * real-time loop where an allocator call may block or synchronise the
 * device, or in a process whose allocator hooks forbid allocation after
 * initialisation. Such a caller passes its own inputs and output; the scratch
 * apt_gather_rows would take as `workspace` is a fixed array built into the
 * library's device image instead (about 12.6 MB, held by every GPU that loads
 * the library until the process exits).
 *
 * Same arguments (minus the workspace) and result as apt_gather_rows, with these differences:
 *  - at most apt_gather_static_max_rows() (1 048 576) rows per call; more
 *    returns APT_ERR_CAPACITY with a message and launches nothing;
 *  - it calls no cudaMalloc, cudaFree or other allocating routine. Every call
 *    looks up the array's device address (cudaGetSymbolAddress) with the
 *    calling thread's device current, so the address is never stale, not even
 *    after the device's context has been torn down and made anew. The first
 *    call on each device makes the CUDA runtime load the library's device
 *    image if it has not yet: make that first call before any stream capture
 *    begins;
 *  - every call on a device uses the same array, which still holds the
 *    previous call's contents (the call clears what has to start at zero).
 *    Two calls that overlap on the GPU — different streams, or different host
 *    threads — race on it: issue them on one stream, or order them yourself.
 */
int64_t apt_gather_static_max_rows(void);
int apt_gather_rows_static(const int64_t* index, int64_t num_rows,
                           const int64_t* feat_pos_map, int64_t num_nodes,
                           const void* dev_feats, int64_t num_dev_rows,
                           int64_t dev_row_bytes, const void* uva_feats,
                           int64_t num_uva_rows, int64_t uva_row_bytes,
                           int64_t uva_col_offset_bytes, void* out,
                           int32_t* status_word, void* stream);

/* ------------------------------------------------------------ SpMM / SDDMM
 * Segment-batched COO operators over sampled blocks: edge e of segment k
 * (coo_offset[k] <= e < coo_offset[k+1]) reads input row input_offset[k]+row[e]
 * and accumulates into output row output_offset[k]+col[e]. Offsets are device
 * arrays of num_segments+1 entries. Take the role of CopyUSumCUDA, CopyESumCUDA,
 * UMulESumCUDA (src/cuda/spmm.cu:7-148; hosts src/spmm.cc:9-42) and UAddVCUDA,
 * UMulVCUDA (src/cuda/sddmm.cu:7-103; hosts src/sddmm.cc:9-31).
 *
 * The output is fully written (rows without edges become 0); it needs no
 * zero-fill. When col is non-decreasing inside every segment (a sampled
 * block), each output row is reduced by one warp in edge order: no atomics,
 * deterministic. Otherwise the edges are first grouped by output row with a
 * counting sort on the device and reduced by the same kernel (no float atomics;
 * the order of the terms inside a row then depends on scheduling).
 * op: 0 copy_u, 1 copy_e, 2 u_mul_e, 3 u_add_e (the arithmetic the reference's
 *     UMulESum kernel actually performs, src/cuda/spmm.cu:78).
 * edata (copy_e, u_mul_e, u_add_e) has num_edges rows of edata_dim columns,
 * edata_dim == feat_dim, or a divisor of feat_dim (one scalar per head,
 * broadcast over feat_dim/edata_dim columns).
 * workspace: apt_spmm_workspace_bytes(num_out_rows, num_edges) bytes.
 */
size_t apt_spmm_workspace_bytes(int64_t num_out_rows, int64_t num_edges);
int apt_spmm_sum(int op, int dtype, const int64_t* coo_row,
                 const int64_t* coo_col, int64_t num_edges, const void* input,
                 const void* edata, int64_t edata_dim, int64_t feat_dim,
                 const int64_t* coo_offset, const int64_t* input_offset,
                 const int64_t* output_offset, int num_segments,
                 int64_t num_out_rows, void* out, void* workspace,
                 size_t workspace_bytes, void* stream);

/* op: 0 u_add_v, 1 u_mul_v; out has num_edges rows of feat_dim columns. */
int apt_sddmm(int op, int dtype, const int64_t* coo_row,
              const int64_t* coo_col, int64_t num_edges, const void* lhs,
              const void* rhs, int64_t feat_dim, const int64_t* coo_offset,
              const int64_t* lhs_offset, const int64_t* rhs_offset,
              int num_segments, void* out, void* stream);

/* Fused GAT edge pipeline over one sampled block whose edges are grouped by
 * destination (col non-decreasing): per destination d and head h,
 *   s_e = leaky_relu(el[row[e], h] + er[d, h]),  a = softmax of s over d's edges,
 *   out[d, h, :] = sum_e a_e * ft[row[e], h, :].
 * It stands for the DGL calls of the reference's SNP-GAT layer
 * (python/npc/model/gatconv.py:113-124: u_add_v, leaky_relu, edge_softmax,
 * u_mul_e + sum), which the reference leaves to DGL. ft is [num_src,
 * num_heads*head_dim], el [num_src, num_heads], er [num_dst, num_heads];
 * out_attn ([num_edges, num_heads], may be NULL) receives a. Rows without
 * edges become 0. Edges that are not grouped set APT_FLAG_NOT_GROUPED and give
 * zeros. workspace: apt_spmm_workspace_bytes(num_dst, 0) bytes. */
int apt_gat_edge_softmax_sum(int dtype, const int64_t* coo_row,
                             const int64_t* coo_col, int64_t num_edges,
                             const void* ft, const void* el, const void* er,
                             int num_heads, int64_t head_dim,
                             float negative_slope, int64_t num_dst, void* out,
                             void* out_attn, void* workspace,
                             size_t workspace_bytes, int32_t* status_word,
                             void* stream);

/* Edge part of the backward pass of apt_gat_edge_softmax_sum (what DGL's autograd
 * runs for python/npc/model/gatconv.py:113-124), same block and layouts. With
 * g = grad_out[d, h, :] ([num_dst, num_heads*head_dim]):
 *   dot_e = <g, ft[row[e], h, :]>,  t = sum over d's edges of a_e dot_e,
 *   grad_s_e = a_e (dot_e - t) * (el[row[e],h] + er[d,h] > 0 ? 1 : negative_slope)
 * out_attn[e, h] = a_e, out_grad_score[e, h] = grad_s_e (both [num_edges, num_heads]),
 * out_grad_er[d, h] = sum_e grad_s_e. The sums over the source side follow as
 * apt_spmm_sum calls with row and col swapped: grad_ft = u_mul_e(grad_out, out_attn),
 * grad_el = copy_e(out_grad_score). workspace: apt_spmm_workspace_bytes(num_dst, 0). */
int apt_gat_edge_backward(int dtype, const int64_t* coo_row, const int64_t* coo_col,
                          int64_t num_edges, const void* ft, const void* el,
                          const void* er, const void* grad_out, int num_heads,
                          int64_t head_dim, float negative_slope, int64_t num_dst,
                          void* out_attn, void* out_grad_score, void* out_grad_er,
                          void* workspace, size_t workspace_bytes,
                          int32_t* status_word, void* stream);

/* ------------------------------------------- SNP virtual nodes (SAGE / GCN)
 * The id arithmetic of the SNP strategy with virtual nodes: neighbour i of
 * local destination i / fanout, owned by rank o, becomes the virtual node
 * o * num_dst + i / fanout.
 *
 * apt_src_to_vir      MapSrctoVir (src/cuda/npc_kernel.cu:71-117; SrcToVir,
 *                     src/sampling.cc:19-34): out_vir[num_src].
 * apt_srcdst_to_vir   MapSrcDsttoVir (src/cuda/npc_kernel.cu:15-70; SrcDsttoVir,
 *                     src/sampling.cc:36-50): out_vir[num_dst + num_src],
 *                     destinations first (owner * num_dst + index), neighbours
 *                     shifted by world_size * num_dst.
 * apt_vir_send_sizes  GetVirSendOffset / GetVirSendOffsetWithDst
 *                     (src/cuda/npc_kernel.cu:119-183) and the size vector
 *                     SPSampleAndShuffle derives from them (src/sampling.cc:86-106,
 *                     permutations of src/core.cc:80-95). out_send_offset (may be
 *                     null): int64[(with_dst ? 3 : 2) * world_size + 1] lower bounds;
 *                     out_send_sizes: per receiver r (ids, unique virtual nodes) or
 *                     (destinations, ids, unique virtual nodes) bound for r.
 *                     num_sorted_dev, num_unique_dev and base_dev (each may be null)
 *                     override num_sorted, num_unique and base on the device.
 * apt_sp_pack_frontier   out[i] = rank * sp_base * num_total_nodes
 *                     + (sorted_vir[i] % num_dst) * num_total_nodes + sorted_ids[i],
 *                     the packed triple of python/npc/sampler.py:296-300.
 * apt_sp_unpack_frontier out_vir = packed / num_total_nodes, out_ori = packed %
 *                     num_total_nodes (src/sampling.cc:128-129, :141-142).
 * The owner function and its arguments are those of apt_bucket_by_owner.
 */
int apt_src_to_vir(const int64_t* src, int64_t num_src, int64_t fanout,
                   int64_t num_dst, const int64_t* min_vids, int world_size,
                   int shuffle_id_offset, int rank, int node_beg, int node_end,
                   int64_t* out_vir, void* stream);
int apt_srcdst_to_vir(const int64_t* dst, int64_t num_dst, const int64_t* src,
                      int64_t num_src, int64_t fanout, const int64_t* min_vids,
                      int world_size, int shuffle_id_offset, int rank,
                      int node_beg, int node_end, int64_t* out_vir, void* stream);
int apt_vir_send_sizes(const int64_t* sorted_nodes, int64_t num_sorted,
                       const int64_t* num_sorted_dev,
                       const int64_t* unique_nodes, int64_t num_unique,
                       const int64_t* num_unique_dev, int world_size,
                       int64_t base, const int64_t* base_dev, int with_dst,
                       int64_t* out_send_offset, int64_t* out_send_sizes,
                       void* stream);
/* The sender side of the hop in one pass (python/npc/sampler.py:255-300 without
 * destinations): with positions = out_perm of apt_bucket_by_owner over the
 * neighbours, out_sorted_vir[positions[i]] = owner(neighbors[i]) * num_dst +
 * i / fanout (the stably sorted virtual ids) and out_packed[positions[i]] = the
 * packed triple of apt_sp_pack_frontier. num_dst_dev (may be null) overrides
 * num_dst on the device; out_count (may be null) receives num_dst * fanout. */
int apt_sp_map_place_pack(const int64_t* neighbors, const int64_t* positions,
                          int64_t num_dst, const int64_t* num_dst_dev,
                          int64_t fanout, const int64_t* min_vids, int world_size,
                          int shuffle_id_offset, int rank, int node_beg,
                          int node_end, int64_t sp_base, int64_t num_total_nodes,
                          int64_t* out_sorted_vir, int64_t* out_packed,
                          int64_t* out_count, void* stream);
int apt_sp_pack_frontier(const int64_t* sorted_vir, const int64_t* sorted_ids,
                         int64_t n, int64_t num_dst, int rank, int64_t sp_base,
                         int64_t num_total_nodes, int64_t* out, void* stream);
int apt_sp_unpack_frontier(const int64_t* packed, int64_t n, const int64_t* n_dev,
                           int64_t num_total_nodes, int64_t* out_vir,
                           int64_t* out_ori, void* stream);

/* ------------------------------------------- dry run: hotness and cache policy
 * The access counters the reference keeps on the host during a dry run
 * (counter[input_nodes.cpu()] += 1, examples/dryrun.py:86-93,
 * python/npc/cost_model/estimator.py:433-436), the order the cache policy sorts
 * them into (torch.sort(freq, descending=True)[1], python/npc/ops.py:189-231,
 * estimator.py:208-209) and the hit volume of a cache of the hottest nodes
 * (get_cache_miss, estimator.py:22-30), kept on the device.
 *
 * apt_hotness_add    counters[ids[i]] += 1 (int32 counters of num_nodes entries).
 * apt_hot_order      out_sorted_idx[num_nodes] = node ids by falling counter; equal
 *                    counters by rising id (the reference's sort leaves ties open).
 * apt_cached_access  out[0] = sum of all counters, out[1] = sum over the first
 *                    num_cache entries of sorted_idx (device int64[2]).
 */
int apt_hotness_add(const int64_t* ids, int64_t n, const int64_t* n_dev,
                    int32_t* counters, int64_t num_nodes, int32_t* status_word,
                    void* stream);
size_t apt_hot_order_workspace_bytes(int64_t num_nodes);
int apt_hot_order(const int32_t* counters, int64_t num_nodes, void* workspace,
                  size_t workspace_bytes, int64_t* out_sorted_idx, void* stream);
int apt_cached_access(const int32_t* counters, int64_t num_nodes,
                      const int64_t* sorted_idx, int64_t num_cache,
                      int64_t* out_total_and_cached, void* stream);

/* out = cat(a[0:na], b[0:nb]) where na / nb come from the device words num_a_dev /
 * num_b_dev when given (num_a / num_b are then upper bounds): the
 * torch.cat((seeds, shuffled_neigh)) of the SNP-GAT sampler
 * (python/npc/sampler.py:230) without a host read. *out_count_dev = na + nb. */
int apt_concat_ids(const int64_t* a, int64_t num_a, const int64_t* num_a_dev,
                   const int64_t* b, int64_t num_b, const int64_t* num_b_dev,
                   int64_t* out, int64_t* out_count_dev, void* stream);

/* ------------------------------------------------------- local row movers
 * out[i] = in[index[i]] and out[index[i]] = in[i] over rows of row_bytes
 * bytes (16-byte vectors when alignment allows). These are the index_select /
 * index_select_backward steps of FeatShuffle (src/feat_shuffle.cc:13-28) for
 * a permutation index, and the h[inverse_idx] step that precedes it
 * (python/npc/model/sage_model.py:67).
 */
int apt_rows_gather(const void* in, const int64_t* index, int64_t num_out_rows,
                    int64_t row_bytes, void* out, void* stream);
int apt_rows_scatter(const void* in, const int64_t* index, int64_t num_in_rows,
                     int64_t row_bytes, void* out, void* stream);

/* ------------------------------------------------ peer-to-peer all-to-all
 * Replaces the grouped ncclSend/ncclRecv all-to-all (_AlltoAll,
 * src/ops/collective.cc:223-266) used by ShuffleSeeds (src/sampling.cc:176-191)
 * and FeatShuffle (src/feat_shuffle.cc:20-22) with stores into the receiving
 * GPU's memory over NVLink.
 *
 * Every rank owns an inbox of 2 (epoch parity) x world_size regions of
 * region_bytes each plus flag words, allocated by apt_p2p_create with
 * cudaMalloc and exported as a CUDA IPC handle. Ranks exchange the 64-byte
 * handles out of band (the host side uses torch.distributed) and map each
 * other's inbox with apt_p2p_attach. One all-to-all is then:
 *   apt_p2p_push   each rank copies its rows for peer r into region [me] of
 *                  r's inbox, fences, and releases flag (epoch, row count);
 *   apt_p2p_wait   a one-block kernel waits (bounded by timeout_ns) for the
 *                  world_size flags of this epoch and writes the received row
 *                  counts to a device array;
 *   apt_p2p_pull   copies / permutes the received rows out of the inbox.
 * All ranks must issue the same sequence of all-to-alls on one stream each.
 * The epoch is kept in the inbox header and advanced by the kernels, so the
 * three calls carry no per-call host state and may be captured in a CUDA graph.
 * Waiting for all flags of epoch e before any store of epoch e+1, together
 * with the parity double buffer, keeps an inbox region from being overwritten
 * before its owner has consumed it.
 */
typedef struct apt_p2p apt_p2p;
#define APT_IPC_HANDLE_BYTES 64

int apt_p2p_create(int rank, int world_size, size_t region_bytes,
                   apt_p2p** out_ctx, void* out_handle /* host, 64 bytes */);
int apt_p2p_attach(apt_p2p* ctx, int peer, const void* handle /* host */);
/* Same-process variant: `base` is the inbox (apt_p2p_local_base) of a context
 * created in this process, e.g. several ranks emulated on one GPU in tests. */
int apt_p2p_attach_ptr(apt_p2p* ctx, int peer, void* base);
void* apt_p2p_local_base(apt_p2p* ctx);
int apt_p2p_destroy(apt_p2p* ctx);
size_t apt_p2p_region_bytes(const apt_p2p* ctx);

/* Push rows. Row j of the outgoing stream (0 <= j < send_offsets[world_size-1])
 * is src row j when src_index is NULL, src row src_index[j] when
 * index_is_dest == 0, and otherwise the src row t with src_index[t] == j
 * (src_index is then a permutation that names each src row's position); rows
 * [send_offsets[r-1], send_offsets[r]) go to peer r. send_offsets is a DEVICE
 * array of world_size inclusive row offsets; max_rows is a host-side upper
 * bound of send_offsets[world_size-1] that sizes the grid. Rows that do not
 * fit a region are dropped and APT_FLAG_TABLE_FULL is set. Advances the epoch.
 * With src_index NULL and index_is_dest == 2 every peer gets the same rows: row l
 * of each peer's bucket is src row l (the all-broadcast of AllBroadcastV2,
 * src/ops/collective.cc:367-402, without the world_size-fold copy of the input). */
int apt_p2p_push(apt_p2p* ctx, const void* src, const int64_t* src_index,
                 int index_is_dest, const int64_t* send_offsets, int64_t max_rows,
                 int64_t row_bytes, int32_t* status_word, void* stream);
/* Wait for this epoch's flags; out_recv_counts int64[world_size + 1] (device)
 * receives the rows each peer sent and, in the last entry, their total.
 * timeout_ns <= 0 selects the default bound: the environment variable
 * APT_P2P_TIMEOUT_MS (read once per process), else 30 s; it must exceed any skew
 * between the ranks that is not a failure. On timeout APT_FLAG_PEER_TIMEOUT is
 * ORed into status_word, the counts of the missing peers are 0, and the inbox is
 * marked unusable: the two-region rotation no longer proves that a peer has read
 * a region before it is written again, so every later apt_p2p_push,
 * apt_p2p_push_direct, apt_p2p_wait and apt_p2p_alltoall_fused on this context
 * stores nothing on any peer and sets APT_FLAG_PEER_TIMEOUT again. Recovery:
 * destroy the contexts of all ranks and create new ones behind a host barrier.
 * (The reference has no counterpart: a lost peer blocks its ncclGroupEnd for good,
 * src/ops/collective.cc:234-249.) */
int apt_p2p_wait(apt_p2p* ctx, int64_t* out_recv_counts, int32_t* status_word,
                 int64_t timeout_ns, void* stream);
/* The default bound above in nanoseconds, and whether a wait of this context
 * has timed out (synchronous 4-byte read of the inbox header). */
int64_t apt_p2p_default_timeout_ns(void);
/* Measurement aid: one cudaMemcpyAsync of nbytes (at most one region) from this
 * rank's inbox into the same place of `peer`'s inbox, i.e. a plain copy over the
 * link the exchange uses; gives the link rate a shuffle is compared with. It
 * overwrites inbox data, so no exchange may be in flight. */
int apt_p2p_probe_copy(apt_p2p* ctx, int peer, size_t nbytes, void* stream);
int apt_p2p_poisoned(apt_p2p* ctx, int* out_poisoned);
/* Copy received rows out of the inbox in peer order (peer 0's rows first).
 * If dst_index is NULL row j of the concatenation lands at dst row j; else if
 * index_is_source it is a gather: dst row i = concatenation row dst_index[i]
 * (num_dst_rows rows); else a scatter: concatenation row j lands at
 * dst_index[j]. recv_counts is the device array apt_p2p_wait filled. Without an
 * index at most num_dst_rows rows of the concatenation are copied (the capacity
 * of dst); with a scatter index every row of the concatenation is visited and a
 * row whose destination lies outside [0, num_dst_rows) is dropped. */
int apt_p2p_pull(apt_p2p* ctx, const int64_t* recv_counts,
                 const int64_t* dst_index, int index_is_source,
                 int64_t num_dst_rows, int64_t max_rows, int64_t row_bytes,
                 void* dst, void* stream);
/* Reduce-scatter epilogue, the receiving half of _AllReduce (one ncclReduce per
 * root, src/ops/collective.cc:404-436) behind MPFeatShuffleFwd
 * (src/feat_shuffle.cc:54-64): after a push in which every rank sent its partial
 * rows for this rank's segment, dst[num_rows x row_elems] = the sum over the
 * peers in rank order (fp32 accumulator; dtype APT_F32 / APT_BF16 / APT_F16).
 * A peer that sent another row count is left out and APT_FLAG_SIZE_MISMATCH set. */
int apt_p2p_pull_sum(apt_p2p* ctx, const int64_t* recv_counts, int dtype,
                     int64_t num_rows, int64_t row_elems, void* dst,
                     int32_t* status_word, void* stream);

/* Direct placement (opt-in): an inbox with landing_slots landing buffers of
 * landing_bytes each behind it. The receiver first sends every sender, with an
 * ordinary apt_p2p_push of 8-byte rows + apt_p2p_wait, the final row slot of each
 * row it is about to get; apt_p2p_push_direct then stores row l for peer r at
 * slot list[r][l] of r's landing buffer `landing_slot`, so that FeatShuffle's
 * index_select / index_select_backward pass over the received rows
 * (src/feat_shuffle.cc:13-28) needs no second kernel. After the apt_p2p_wait
 * that follows, apt_p2p_landing(ctx, landing_slot) holds the result; it stays
 * valid until that landing buffer is named again. All ranks must create their
 * inboxes with the same sizes. Slots outside the buffer set APT_FLAG_TABLE_FULL. */
int apt_p2p_create_landing(int rank, int world_size, size_t region_bytes,
                           size_t landing_bytes, int landing_slots,
                           apt_p2p** out_ctx, void* out_ipc_handle);
size_t apt_p2p_landing_bytes(const apt_p2p* ctx);
void* apt_p2p_landing(apt_p2p* ctx, int landing_slot);
int apt_p2p_push_direct(apt_p2p* ctx, const void* src, const int64_t* src_index,
                        int index_is_dest, const int64_t* send_offsets,
                        int64_t max_rows, int64_t row_bytes, int landing_slot,
                        int32_t* status_word, void* stream);

/* The same all-to-all as push + wait + pull, as ONE cooperative kernel in which
 * the local pass (moving received rows to their final place) overlaps the
 * NVLink transfer: buckets are cut into `chunks` (1..8) row ranges, each with
 * its own flag; blocks push chunk c+1 while they pull chunk c. The receiver has
 * to know how many rows every source sends (recv_offsets, device, inclusive),
 * which FeatShuffle and AlltoAll do (their offsets come from the host). Rows
 * must be multiples of 16 bytes. pull_index NULL: dst row j = concatenation row
 * j; else dst row i = concatenation row pull_index[i] (num_dst_rows rows). */
int apt_p2p_alltoall_fused(apt_p2p* ctx, const void* src, const int64_t* src_index,
                           int index_is_dest, const int64_t* send_offsets,
                           const int64_t* recv_offsets, const int64_t* pull_index,
                           int64_t num_dst_rows, int64_t row_bytes, int chunks,
                           void* dst, int32_t* status_word, int64_t timeout_ns,
                           void* stream);

/* --------------------------------------------------------- setup utilities
 * Not on the timed path; they prepare the synthetic graphs of the benchmark
 * on the GPU so that a 1.6 G-edge graph is built in seconds. */

/* R-MAT edge list: edge e draws its (src, dst) bits from Philox4x32-10 keyed
 * by `seed`, counter (e, attempt); endpoints >= num_nodes are redrawn. */
int apt_rmat_edges(uint64_t seed, int64_t first_edge, int64_t num_edges,
                   int scale, int64_t num_nodes, float a, float b, float c,
                   int64_t* out_src, int64_t* out_dst, void* stream);
/* Zipf(s) ranks in [1, num_ranks] for skewed seed streams: draw i is
 * floor((1 + u ((N+1)^(1-s) - 1))^(1/(1-s))) with u from Philox keyed by `seed`
 * at counter first_draw + i (rank k has the mass of x^-s over [k, k+1)). */
int apt_zipf_ranks(uint64_t seed, int64_t first_draw, int64_t num_draws,
                   int64_t num_ranks, double s, int64_t* out, void* stream);
/* Ascending radix sort (cub) of the low `end_bit` bits of uint64 keys from
 * keys_in into keys_out. temp: apt_sort_u64_temp_bytes(n) bytes. */
size_t apt_sort_u64_temp_bytes(int64_t n);
int apt_sort_u64(const uint64_t* keys_in, uint64_t* keys_out, int64_t n,
                 void* temp, size_t temp_bytes, int end_bit, void* stream);
/* Standard-normal rows: element (row, col) from Philox keyed by seed; written
 * as dtype. Output row r holds node row_ids[r], or first_row + r when row_ids
 * is NULL, so a cache table and the full table agree row by row. */
int apt_normal_rows(uint64_t seed, int64_t first_row, const int64_t* row_ids,
                    int64_t num_rows, int64_t dim, int dtype, void* out,
                    void* stream);

#ifdef __cplusplus
}
#endif
#endif /* APT_B200_H_ */
