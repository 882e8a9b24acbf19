/* C ABI of libtilefusion_b200: fused sparse-dense chains on one B200 (sm_100a).
 *
 *   GeMM-SpMM   D = A * (B * C)      A sparse CSR, B and C dense
 *   SpMM-SpMM   D = A * (B * C)      A and B sparse CSR, C dense
 *   SDDMM-SpMM  D = (A .* (Q K^T)) * V
 *
 * Plain pointers and sizes only.  CSR: int32 row pointers / column indices,
 * fp32 values, sorted columns.  Dense: row-major fp32.  Every function returns
 * TF_OK or a negative error code; tf_last_error() gives the message of the
 * calling thread's last failure.  There is no CPU fallback: executors fail
 * with TF_ERR_CUDA when no sm_100 device is usable.
 *
 * Each entry point names the interface of the reference project
 * (SwiftWare-Lab/tile-fusion) it stands in for; paths are inside that project.
 */
#ifndef TILE_FUSION_B200_H
#define TILE_FUSION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TF_OK = 0,
  TF_ERR_ARG = -1,         /* null pointer, bad size, unsorted columns, ...           */
  TF_ERR_UNSUPPORTED = -2, /* a combination the library does not implement             */
  TF_ERR_CUDA = -3,        /* CUDA runtime error (message holds cudaGetErrorString)    */
  TF_ERR_TIMEOUT = -4,     /* a bounded in-kernel wait ran out; results are not valid  */
  TF_ERR_NOMEM = -5
} tf_status;

const char *tf_last_error(void);
const char *tf_version(void);

/* ------------------------------------------------------------------------- */
/* Inspector: reference-format schedule                                       */
/* ------------------------------------------------------------------------- */

/* Which reference inspector to reproduce bit for bit. */
typedef enum {
  /* SparseFusionInspector::generateFusedScheduleForAllFused
   *   fusion/include/sparse-fusion/Fusion_Inspector.h:32 (fixed tiles) */
  TF_INSPECT_FIXED = 1,
  /* InspectorForTileFusedCSRVariableTileSize::generateVariableTileSizeScheduleForBothWavefronts
   *   Fusion_Inspector.h:676 (SpMM-SpMM, cache budget) */
  TF_INSPECT_VT_SPMM = 2,
  /* ...::generateVariableTileSizeScheduleGeMMSpMM  Fusion_Inspector.h:851 */
  TF_INSPECT_VT_GEMM = 3,
  /* ...::generateVariableTileSizeSchedule  Fusion_Inspector.h:542 (wave 2 split over threads) */
  TF_INSPECT_VT_SPMM_THREADS = 4
} tf_inspect_kind;

/* Mirrors sym_lib::ScheduleParameters (fusion/include/sparse-fusion/Fusion_Defs.h:21-55)
 * plus the arguments the variable-tile inspectors take. */
typedef struct {
  int kind;               /* tf_inspect_kind                                          */
  int num_threads;        /* _num_threads                                             */
  int iter_per_partition; /* IterPerPartition (TF_INSPECT_FIXED)                      */
  int tile_m;             /* TileM: cache budget in bytes (variable-tile kinds)       */
  int b_cols;             /* BCol: dense width of the first product                   */
  int c_cols;             /* CCol (TF_INSPECT_VT_GEMM)                                */
  int data_size;          /* DataSize: bytes per value, 4 for fp32                    */
} tf_sched_params;

/* The schedule: sym_lib::MultiDimensionalSet
 *   (fusion/include/sparse-fusion/MultiDimensionalSet.h:15-25), the README's FusedSchedule. */
typedef struct tf_schedule tf_schedule;

/* Runs one of the reference inspectors on the pattern of A (m x m).
 * Rejects (TF_ERR_ARG) inputs on which the reference divides by zero or never ends. */
int tf_inspect(int m, const int *Ap, const int *Ai, const tf_sched_params *p, tf_schedule **out);

/* n1 = levels, n_parts = ptr1[n1], n_ids = ptr2[n_parts], has_ker = ker_begin present. */
int tf_schedule_dims(const tf_schedule *s, int *n1, int *n_parts, int *n_ids, int *has_ker);
/* Borrowed pointers into the schedule: ptr1[n1+1], ptr2[n_parts+1], id[n_ids], type[n_ids],
 * ker_begin[2*n_parts] (NULL when absent).  Any argument may be NULL. */
int tf_schedule_arrays(const tf_schedule *s, const int **ptr1, const int **ptr2, const int **id,
                       const int **type, const int **ker_begin);
/* stats[0..4] = fused rows, fused nnz, tile-size mean, tile-size std, partitions
 * (the values the reference writes into Stats::OtherStats, Fusion_Inspector.h:671,1013,1049). */
int tf_schedule_stats(const tf_schedule *s, double stats[5]);
/* Builds a schedule object from caller arrays (copied), e.g. one produced elsewhere. */
int tf_schedule_from_arrays(int n1, const int *ptr1, const int *ptr2, const int *id, const int *type,
                            const int *ker_begin, tf_schedule **out);
/* Flat int32 image of a schedule, so inspection can be paid once and reused
 * (the reference keeps the schedule across epochs, FusedGCNModule.py:10). */
int tf_schedule_serialized_size(const tf_schedule *s, size_t *n_ints);
int tf_schedule_serialize(const tf_schedule *s, int *buf, size_t n_ints);
int tf_schedule_deserialize(const int *buf, size_t n_ints, tf_schedule **out);
void tf_schedule_free(tf_schedule *s);

/* ------------------------------------------------------------------------- */
/* Device plan                                                                */
/* ------------------------------------------------------------------------- */

typedef struct {
  int m, n;          /* rows, columns                                                  */
  const int *ap;     /* m + 1                                                          */
  const int *ai;     /* ap[m]                                                          */
  const float *ax;   /* ap[m]                                                          */
} tf_csr;            /* host memory */

typedef enum {
  TF_MODE_STREAM = 0,   /* one persistent launch; the intermediate lives in an L2-sized ring */
  TF_MODE_SCHEDULE = 1, /* follow a reference-format schedule tile by tile (two waves)       */
  TF_MODE_UNFUSED = 2   /* two full passes, intermediate through HBM (self-check baseline)   */
} tf_exec_mode;

typedef struct {
  int mode;               /* tf_exec_mode                                               */
  int rows_per_block;     /* rows per work item, 0 = default                            */
  int ring_bytes;         /* budget for the intermediate ring, 0 = default, <0 = no ring */
  int slack_blocks;       /* producer lead over consumers in blocks, <0 = default       */
  int ctas_per_sm;        /* 0 = as many as fit                                         */
  int halo_rows;          /* rows of the intermediate that arrive from elsewhere and are
                             appended after the m local rows (multi-GPU); 0 otherwise   */
  int n_boundary;         /* number of entries of `boundary_rows`                       */
  const int *boundary_rows; /* local intermediate rows other ranks need first (sorted)  */
  int tile_slots;         /* gather tiles: dense-row segments (128 B) a tile may stage in shared
                             memory; 0 = default, <0 = never tile (gather from global memory)      */
  int tile_max_bz;        /* gather tiles: most grid planes a tile may span, 0 = default           */
  int tile_double_buffer; /* gather tiles: >0 = tiles sized to half the staging buffer so that the copies of
                             the next column chunk overlap the current one, <0 = full-size tiles, 0 = default */
  int tensor_cores;       /* GeMM-SpMM dense producer: 0 = tcgen05 3xTF32 when the shape allows
                             (K % 4 == 0, N % 16 == 0, N <= 256), <0 = always the fp32 CUDA-core tile */
  int tile_pipeline;      /* SpMM-SpMM with both operators tiled and no ring requested: 0 = run the tiles on
                             the role-split pipeline (one CTA per SM: staging warps copy the next column
                             chunk while compute warps work on the current one), <0 = never              */
  int lattice_march;      /* SpMM-SpMM whose two operators are star stencils on one 3-D grid in natural order
                             (every nonzero names the row's own grid point or one of its six neighbours):
                             0 = run the plane-marching kernel, which keeps the intermediate in shared memory,
                             <0 = never (general CSR path).  GeMM-SpMM plans on such an operator use the same
                             kernel as the consumer of the tensor-core producer's rows (0) or the ticket executor (<0) */
  int exchange;           /* tf_multi_plan only: 0 = halo rows are written by the copy engines straight into the
                             neighbours' memory (CUDA IPC) where every rank is a process of its own on one host,
                             else ncclSend / ncclRecv; <0 = always ncclSend / ncclRecv (every rank must say the same) */
} tf_plan_opts;

typedef struct tf_plan tf_plan;

/* SpMM-SpMM plan for D = A*(B*C); B == NULL means B = A.  `n_cols` = columns of C and D.
 * `sched` is required for TF_MODE_SCHEDULE and ignored otherwise.
 * Stands in for the analysis step of the reference's bench classes
 * (fusion/example/SpMM_SpMM_SP_Demo_Utils.h:165-199). */
int tf_plan_spmm_spmm(const tf_csr *A, const tf_csr *B, int n_cols, const tf_plan_opts *o,
                      const tf_schedule *sched, tf_plan **out);
/* GeMM-SpMM plan for D = A*(B*C), B m x k dense, C k x n_cols dense. */
int tf_plan_gemm_spmm(const tf_csr *A, int k, int n_cols, const tf_plan_opts *o,
                      const tf_schedule *sched, tf_plan **out);
/* SDDMM-SpMM plan: D = (A .* (Q K^T)) V, Q,K m x kq, V m x nv. */
int tf_plan_sddmm_spmm(const tf_csr *A, int kq, int nv, const tf_plan_opts *o, tf_plan **out);
void tf_plan_free(tf_plan *p);

/* Host-only preview of the stream plan the library would run (no device needed): `items_out`
 * receives a malloc'd array of 8 ints per item {kind, block, row_begin, row_end, need, base, aux0,
 * aux1} in ticket order (release with tf_free); info = {items, producer blocks, consumer blocks,
 * ring rows, begin of phase 1, begin of phase 2, end, intermediate rows}.  `resident_ctas` is the
 * number of CTAs assumed resident (it sets the default slack).  No counterpart in the reference. */
int tf_plan_preview(const tf_csr *A, const tf_csr *B, int producer_is_gemm, int n_cols,
                    const tf_plan_opts *o, int resident_ctas, int **items_out, long long *n_items,
                    long long info[8]);
void tf_free(void *p);
/* Host-only: the gather tiles the library would build for operator A.  Arrays are malloc'd
 * (tf_free): row_ptr[n_tiles+1] into rows[], halo_ptr[n_tiles+1] into halo[] (staged source rows in
 * slot order).  n_tiles = 0 when tiling is declined.  info = {bx, by, bz, 1000 * nonzeros per staged
 * row}.  No counterpart in the reference. */
int tf_tiling_preview(const tf_csr *A, int tile_slots, int tile_max_bz, int **row_ptr, int **rows,
                      int **halo_ptr, int **halo, int *n_tiles, int info[4]);
/* Host-only: how the library sees operator A (m x n CSR, of which the last `halo_rows` columns are halo rows
 * appended after the local ones) as a star stencil on a 3-D grid in natural order -- the form the
 * plane-marching executor runs from.  info = {recognised, nx, ny, nz, source planes below, source planes above,
 * classes, 0}.  When recognised: dict = (classes + 1) x 8 floats, one coefficient vector per class in
 * sorted-column order {z-, y-, x-, centre, x+, y+, z+, 0} (the last class is all zero); patch_cls =
 * nz x ceil(ny/2) x ceil(nx/2) words holding the classes of the rows (2px+dx, 2py+dy, z) in byte 2*dy+dx;
 * items = n_items x {x0, y0, z begin, z end, first column, flags}, the executor's work list for `n_cols`
 * dense columns on `ctas` resident CTAs.  Arrays are malloc'd (tf_free).  No counterpart in the reference. */
int tf_lattice_preview(const tf_csr *A, int halo_rows, int n_cols, int ctas, int info[8], float **dict,
                       unsigned **patch_cls, int **items, int *n_items);
/* info = {bx, by, bz, tiles} of the first operator's gather tiles, then the same for the second
 * operator's (zeros where an operator is not tiled). */
int tf_plan_tile_info(const tf_plan *p, int info[8]);

/* info[0] items, [1] producer blocks, [2] consumer blocks, [3] ring rows (0 = full-size
 * intermediate), [4] grid CTAs, [5] threads per CTA, [6] kernels launched by the last call,
 * [7] intermediate rows allocated. */
int tf_plan_info(const tf_plan *p, long long info[8]);
/* Number of polls (each followed by a short sleep) after which an in-kernel wait on another
 * block's completion gives up, sets the plan's error status and lets the kernel return.
 * Default 1 << 22 (of the order of a second). */
int tf_plan_set_wait_limit(tf_plan *p, int polls);
/* Waits for the plan's work on `stream` and reports TF_ERR_TIMEOUT if a bounded wait ran out. */
int tf_plan_status(tf_plan *p, void *stream);

/* ------------------------------------------------------------------------- */
/* Executors, device pointers.  `stream` is a cudaStream_t (NULL = default).   */
/* D is overwritten.  These calls only enqueue work: a bounded in-kernel wait  */
/* that ran out is sticky in the plan and is reported (and cleared) by         */
/* tf_plan_status, which callers of the device path should ask once per batch. */
/* ------------------------------------------------------------------------- */

/* spmmCsrSpmmCsrFusedVectorized2_32SP (fusion/src/SpMM_SpMM_vectorized.cpp:876) and its scalar
 * form spmmCsrSpmmCsrFused<float> (fusion/src/SpMM_SpMM.cpp:211). */
int tf_exec_spmm_spmm(tf_plan *p, const float *C, float *D, void *stream);

/* forwardForOneLayerFusedParallelSeparatedVectorizedSP
 * (fusion/gcn/GCN_Layer_MKL_Forward_Utils.h:218; weight k x n) and, with w_transposed != 0,
 * the scalar / torch-binding layout weight n x k (ibid. :182; binding-project/src/Functions.cpp:629).
 * relu != 0 applies max(0, .) to D (binding-project/gcn-e2e-training/FusedGCNModule.py:16). */
int tf_exec_gemm_spmm(tf_plan *p, const float *B, const float *W, int w_transposed, int relu, float *D,
                      void *stream);

/* SDDMM as defined by sddmm_cpu (codegen/triton/sddmm.py:173) followed by the CSR SpMM
 * (fusion/src/SpMM_SpMM.cpp:20); the sampled matrix is never stored. */
int tf_exec_sddmm_spmm(tf_plan *p, const float *Q, const float *K, const float *V, float *D,
                       void *stream);

/* Multi-GPU phases of a plan built with boundary_rows / halo_rows:
 *   phase 0  produce the boundary rows of the intermediate (then send them),
 *   phase 1  everything that needs no halo row,
 *   phase 2  the consumer rows that read halo rows (after the receive).
 * tf_plan_intermediate gives the device buffer: local rows first, then halo rows. */
int tf_exec_phase(tf_plan *p, int phase, const float *in0, const float *in1, int w_transposed, int relu,
                  float *D, void *stream);
int tf_plan_intermediate(tf_plan *p, float **dev_ptr, long long *rows, int *cols);
/* Device buffers of the halo exchange: `send` holds the boundary rows in the order of
 * boundary_rows (filled by phase 0), `halo` is where received rows go (the tail of the
 * intermediate).  No counterpart in the reference, which runs on one shared-memory host. */
int tf_plan_exchange_buffers(tf_plan *p, float **send, long long *send_rows, float **halo,
                             long long *halo_rows);

/* ------------------------------------------------------------------------- */
/* Several GPUs: one process (or thread) per GPU, rows of A split in consecutive */
/* blocks, halo rows of the intermediate exchanged over NCCL.  No counterpart in */
/* the reference, which runs on one shared-memory host.  NCCL (libnccl.so.2) is  */
/* looked up in the process at run time; TF_ERR_UNSUPPORTED when it is absent.   */
/* ------------------------------------------------------------------------- */
typedef struct tf_comm tf_comm;
typedef struct tf_multi tf_multi;
/* Rank 0 makes an id (ncclGetUniqueId) and hands it to the other ranks by any means; every rank then joins with
 * the device that is current in the calling thread.  tf_comm_from_nccl adopts an ncclComm_t the caller already
 * has (it is not destroyed by tf_comm_free). */
int tf_comm_unique_id(char id[128]);
int tf_comm_create(const char id[128], int world, int rank, tf_comm **out);
int tf_comm_from_nccl(void *nccl_comm, int world, int rank, tf_comm **out);
void tf_comm_free(tf_comm *c);
/* Plan for this rank's rows [r0, r1) of the global operator A; `ai` holds GLOBAL column ids; the ranks' ranges must
 * be consecutive in rank order.  chain 0 = SpMM-SpMM D = A*(A*C), chain 1 = GeMM-SpMM D = A*(B*C) (k = columns of
 * B).  A collective: every rank of the communicator calls it (the halo lists are all-gathered), then holds
 *   - the partition arrays: halo = sorted column ids outside [r0, r1), boundary = own rows some other rank's halo
 *     names, one send and one receive segment per neighbour (tf_partition_layout gives the same arrays on the host);
 *   - a device plan (tf_plan) with those halo rows and boundary rows. */
int tf_multi_plan(tf_comm *c, int chain, long long r0, long long r1, const int *ap, const long long *ai, const float *ax,
                  int k, int n_cols, const tf_plan_opts *opts, tf_multi **out);
void tf_multi_free(tf_multi *m);
/* info = {local rows, halo rows, boundary rows, first row of C the rank reads, rows of C it reads (SpMM-SpMM: own
 * rows plus ghost rows, one contiguous range), send peers, receive peers, threads per CTA of the executor}. */
int tf_multi_info(const tf_multi *m, long long info[8]);
tf_plan *tf_multi_plan_handle(tf_multi *m);
/* One step on this rank, enqueued on `stream` and on the plan's own communication stream: phase 0 (boundary rows of
 * the intermediate), ncclSend / ncclRecv of those rows, phase 1 beside the exchange, phase 2 after the receive.
 * in0 = the rank's rows of C (rows [info[3], info[3] + info[4])) or of B; in1 = the weight (GeMM-SpMM) or NULL. */
int tf_multi_exec(tf_multi *m, const float *in0, const float *in1, int w_transposed, int relu, float *D, void *stream);
/* Waits for the step's work and reports TF_ERR_TIMEOUT if a bounded wait ran out. */
int tf_multi_status(tf_multi *m, void *stream);
/* Step tracing (the reference times its executors with a wall clock around execute(), SWTensorBench.h; a step here
 * spans two streams).  on != 0: following steps record CUDA events around their phases.  ms (may be NULL) receives
 * the last traced step's times in milliseconds from its start: {phase 0 done, exchange done, phase 2 done,
 * phase 1 done, step done}; -1 where nothing was recorded.  Synchronises the device when ms is given. */
int tf_multi_trace(tf_multi *m, int on, float ms[5]);
/* Host only: the partition arrays of `rank` from every rank's bounds and halo list (halo_ptr[world + 1] into
 * halo_ids).  malloc'd (tf_free): boundary_rows (local ids); recv and send as {peer, start, count, contiguous}
 * quadruples, start/count in rows of the halo buffer / of the send buffer. */
int tf_partition_layout(int rank, int world, const long long *bounds, const long long *halo_ptr,
                        const long long *halo_ids, long long **boundary_rows, long long *n_boundary,
                        long long **recv, int *n_recv, long long **send, int *n_send);

/* ------------------------------------------------------------------------- */
/* Executors, host pointers: the README-level calls                            */
/*   swiftware::fusion::spMMSpMMExecutor / geMMSpMMExecutor (README.md:31-32)  */
/* Copies the dense operands to the device, runs, copies D back.              */
/* ------------------------------------------------------------------------- */
int tf_spmm_spmm_host(tf_plan *p, const float *C, float *D);
int tf_gemm_spmm_host(tf_plan *p, const float *B, const float *W, int w_transposed, int relu, float *D);
int tf_sddmm_spmm_host(tf_plan *p, const float *Q, const float *K, const float *V, float *D);

/* Plain CSR SpMM  out = A * X  on device pointers (spmmCsrParallel<float>,
 * fusion/src/SpMM_SpMM.cpp:37, with beta = 0). */
int tf_spmm_dev(const int *Ap, const int *Ai, const float *Ax, int m, const float *X, int n_cols,
                float *out, void *stream);

/* The dense producer alone: T = B * W on device pointers, B m x K, W K x N (N x K when w_transposed),
 * on the tcgen05 tensor cores with the 3xTF32 split (fp32 accuracy).  Needs K % 4 == 0, N % 16 == 0,
 * N <= 256 (TF_ERR_UNSUPPORTED otherwise).  Waits for completion.  Stands in for the per-tile
 * cblas_sgemm of the reference (fusion/gcn/GCN_Layer_MKL_Forward_Utils.h:233). */
int tf_gemm_tc_dev(const float *B, const float *W, int w_transposed, int m, int K, int N, float *T, void *stream);

/* SpMM-SpMM, D = A * (A * C), for callers that cannot allocate device memory.
 *
 * Has no counterpart in the reference.  It is meant for host code that is not allowed to call
 * cudaMalloc / cudaFree at the point where it needs the product: those calls take the driver's
 * allocator lock and may synchronise the whole device, which a request loop that has finished its
 * warm-up, or a component living under somebody else's memory-pool policy, cannot afford.  This
 * entry point therefore calls no allocating routine at all: A (m x m CSR), C and D (m x n_cols,
 * row-major) are DEVICE pointers the caller already owns, and the intermediate A*C is kept in an
 * array that is part of the library image -- tf_noalloc_max_floats() floats (4 Mi = 16 MiB),
 * resident on every GPU that loads the library until the process ends.
 *
 * Limits and rules:
 *  - m * n_cols must not exceed tf_noalloc_max_floats(); larger problems get TF_ERR_ARG with a
 *    message naming the limit (use a plan instead).
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and remembers it; make that first call before any stream capture begins.
 *  - All calls share the one array and it keeps whatever the last call left there.  Each call
 *    rewrites every row it later reads, so nothing needs clearing, but two calls whose kernels
 *    overlap on the GPU (different streams, no ordering between them) race on it.
 *  - Work is enqueued on `stream` (cudaStream_t, NULL = default); the call does not wait for it.  */
int tf_spmm_spmm_noalloc(const int *Ap, const int *Ai, const float *Ax, int m, const float *C, int n_cols,
                         float *D, void *stream);
long long tf_noalloc_max_floats(void);

/* ------------------------------------------------------------------------- */
/* Reordered layouts and orderings (host only)                                */
/* ------------------------------------------------------------------------- */
/* The rows of the second wave of a two-wave schedule as a CSR of their own, in schedule order: createUnfusedData
 * (fusion/example/SpMM_SpMM_SP_Demo_Utils.h:600-636).  malloc'd (tf_free): uf_ap[n_rows + 1], uf_ai, uf_ax. */
int tf_schedule_unfused_csr(const tf_schedule *s, int m, const int *ap, const int *ai, const float *ax, int **uf_ap, int **uf_ai,
                            float **uf_ax, int *n_rows);
/* All rows of A in the order the schedule visits them in its second loop, with the old row of every new row (l2_ptr)
 * and the re-based per-partition pointers (new_mix[2 * (partitions + 1)]): createReorderedAdj
 * (fusion/gcn/SingleLayer/GCN_Single_Layer_SP_Demo_Utils.h:618-653).  malloc'd (tf_free). */
int tf_schedule_reordered_adj(const tf_schedule *s, int m, const int *ap, const int *ai, const float *ax, int **r_ap, int **r_ai,
                              float **r_ax, int **l2_ptr, int **new_mix, int *n_mix);
/* Reverse Cuthill-McKee ordering of the symmetrised pattern, perm[new] = old (caller-allocated, m entries), and
 * B = P A P^T with sorted columns (caller-allocated b_ap[m + 1], b_ai / b_ax[ap[m]]).  Stands in for the METIS
 * reordering front-end of the reference (get_reorderd_matrix, fusion/src/Fusion_Utils.cpp:181-203): a
 * bandwidth-reducing order brings the columns of a row next to the row, which raises the share of rows both the
 * reference's criterion and this library's gather tiles can fuse. */
int tf_rcm_order(int m, const int *ap, const int *ai, int *perm);
int tf_permute_csr(int m, const int *ap, const int *ai, const float *ax, const int *perm, int *b_ap, int *b_ai, float *b_ax);

/* ------------------------------------------------------------------------- */
/* Matrix files                                                               */
/* ------------------------------------------------------------------------- */
/* Reads a sparse matrix file into CSR (int32 indices, fp32 values, sorted columns; arrays malloc'd, tf_free):
 *   *.mtx   Matrix Market coordinate format, real / integer / pattern, general / symmetric / skew-symmetric
 *           (expand_symmetric != 0 mirrors the stored triangle, as the demos' make_full does); duplicates add up;
 *   *.smtx  the DLMC text format: "rows, cols, nnz", row pointers, column indices; every value 1.
 * Stands in for get_matrix_from_parameter / readSparseMatrix (fusion/src/Fusion_Utils.cpp:205-272), which exit
 * the process on a bad file; here a bad file is TF_ERR_ARG / TF_ERR_UNSUPPORTED with a message. */
int tf_read_matrix(const char *path, int expand_symmetric, int *m, int *n, long long *nnz, int **ap, int **ai,
                   float **ax);
/* Dense matrix from a Matrix Market array file (the feature matrices of the GCN demos,
 * get_dense_matrix_from_parameter, Fusion_Utils.cpp:274-283), returned row-major (malloc'd, tf_free). */
int tf_read_dense_mtx(const char *path, int *rows, int *cols, float **data);

/* Counter-based seeded fills on the device: uniform[-1,1) is bit-identical to the host
 * generator, N(0, sigma^2) (Box-Muller) agrees with it to float rounding of log/cos;
 * `offset` is the index of the first element. */
int tf_fill_uniform(float *dev, long long count, unsigned long long seed, long long offset, void *stream);
int tf_fill_normal(float *dev, long long count, unsigned long long seed, long long offset, float sigma,
                   void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TILE_FUSION_B200_H */
