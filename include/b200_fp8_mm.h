/*
 * C ABI of the B200 (sm_100a) FP8 block-scaled GEMM library, libb200fp8mm.so.
 *
 * The operator computed is the one behind the reference's
 * `custom_kernel((a, b, a_scale, b_scale, c)) -> c`
 * (1-amd-fp8-mm/amd-fp8-mm-submission.py:594-604):
 *
 *   c[i,j] = bf16( sum_kb ( sum_{kk in 128-block kb} a[i,kk]*b[j,kk] )
 *                        * a_scale[i,kb] * b_scale[(j + n_phase)/128, kb] )
 *
 * with a, b in e4m3fn, the inner sum accumulated in fp32 from zero by the
 * tensor cores, and the scaled blocks accumulated in fp32
 * (1-amd-fp8-mm/amd-fp8-mm-submission.py:302-357 is the reference loop).
 *
 * Every entry point takes plain pointers and sizes. No entry point ever calls
 * cudaMalloc or cudaFree: scratch for split-K plans is a workspace the caller
 * supplies. The library's device image does carry one fixed 8 MiB array (used only
 * by b200_fp8_mm_static_scratch), which the CUDA runtime materialises on each GPU
 * when the module is loaded there, i.e. during the first call of any entry point on
 * that GPU; make one warm-up call per device at start-up (outside stream capture) to
 * keep module load and address lookup out of latency-critical code.
 *
 * Host-side state: per-device facts looked up once and a cache of encoded TMA
 * tensor maps keyed by (pointer, extents, strides, box); both are guarded by a
 * mutex, so the entry points may be called from several host threads.
 */
#ifndef B200_FP8_MM_H_
#define B200_FP8_MM_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes. 0 is success; everything else means no kernel was launched,
 * except B200_FP8_MM_ERR_LAUNCH (the launch itself failed). */
enum {
  B200_FP8_MM_OK = 0,
  B200_FP8_MM_ERR_NULL = 1,        /* a required pointer is NULL                   */
  B200_FP8_MM_ERR_SHAPE = 2,       /* M, N or K <= 0, or K not a multiple of 128   */
  B200_FP8_MM_ERR_STRIDE = 3,      /* a stride the TMA path cannot address         */
  B200_FP8_MM_ERR_ALIGN = 4,       /* a or b not 16-byte aligned                   */
  B200_FP8_MM_ERR_PHASE = 5,       /* n_phase outside [0,128) or not a multiple of 32 */
  B200_FP8_MM_ERR_WORKSPACE = 6,   /* workspace missing or too small for the plan  */
  B200_FP8_MM_ERR_PLAN = 7,        /* a forced plan is not one the kernels support */
  B200_FP8_MM_ERR_DRIVER = 8,      /* tensor-map encode failed / no sm_100 device  */
  B200_FP8_MM_ERR_LAUNCH = 9,      /* cudaLaunchKernelEx returned an error         */
  B200_FP8_MM_ERR_SCRATCH_LIMIT = 10 /* b200_fp8_mm_static_scratch: the plan needs more
                                        than the scratch built into the library     */
};

/* Device-side status word values (written to device_status[0]; [1] holds the
 * role and barrier that gave up, [2] the block index, [3] the barrier phase). A
 * kernel never traps and never spins without limit: a wait that expires (2 s)
 * records one of these and every role leaves its loop. After a
 * B200_FP8_MM_DEV_WAIT_EXPIRED the output is not valid and a split-K launch may
 * have left the workspace's tile counters mid-count: zero the workspace's first
 * 4096 bytes (and device_status) before the next call that uses them. */
enum {
  B200_FP8_MM_DEV_OK = 0,
  B200_FP8_MM_DEV_WAIT_EXPIRED = 1
};

/* Tile and launch parameters chosen for one problem. Replaces the reference's
 * exact-shape dispatch table (1-amd-fp8-mm/amd-fp8-mm-submission.py:528-578)
 * and its older size heuristic (1-amd-fp8-mm/1-amd-fp8-mm-original.py:484-514). */
typedef struct b200_fp8_mm_plan {
  int block_m;    /* rows of C per CTA (128)                                        */
  int block_n;    /* columns of C per tile: 64, 128, 192 or 256                     */
  int cta_pair;   /* 1: two CTAs share a 256-row tile through cta_group::2          */
  int split_k;    /* number of K ranges per split tile (1 = no tile is split; the
                     selector uses at most 16, a forced plan at most 64)            */
  int stages;     /* depth of the TMA -> shared memory ring                         */
  int grid;       /* CTAs launched (persistent; a multiple of 2 when cta_pair)      */
  int tiles;      /* output tiles (x split_k = work items)                          */
  int smem_bytes; /* dynamic shared memory per CTA                                  */
  int store_bufs; /* staging buffers per warpgroup for the TMA store of c: 1 .. 4 (one per
                     32-column box of the warpgroup's share stages the whole tile at once);
                     0 = plain stores (every tile split, or forced with -1)          */
  int full_tiles; /* output: tiles [0, full_tiles) run whole, the rest (the tail of a
                     partly filled last wave, or all tiles when there are few) are
                     split split_k ways along K                                     */
} b200_fp8_mm_plan;

/*
 * The GEMM. Replaces the pybind launcher `fp8_mm(a, b, as, bs, c, c_tmp)`
 * (1-amd-fp8-mm/amd-fp8-mm-submission.py:8, 514-579).
 *
 *  a        e4m3fn [M,K], element (i,kk) at a + i*lda + kk   (K contiguous)
 *  b        e4m3fn [N,K], element (j,kk) at b + j*ldb + kk
 *  a_scale  fp32, element (i,kb)  at a_scale + i*sa_m + kb*sa_k
 *  b_scale  fp32, element (jb,kb) at b_scale + jb*sb_n + kb*sb_k, with
 *           jb = (j + n_phase)/128: n_phase is the offset of column 0 of this
 *           (shard of) b inside its 128-column scale block, 0 for a whole matrix
 *  c        bf16 [M,N], element (i,j) at c + i*ldc + j; written, never read
 *  lda, ldb multiples of 16; a and b 16-byte aligned (TMA rules)
 *  workspace / workspace_bytes
 *           at least b200_fp8_mm_workspace_bytes(M,N,K) bytes (for a forced plan:
 *           b200_fp8_mm_plan_workspace_bytes), 256-byte aligned;
 *           its first 4096 bytes must be zero before the first call and are left
 *           zero by every call. May be NULL when that function returns 0.
 *  device_status  int[4] in device memory, zeroed by the caller; see the enum above
 *  stream   a cudaStream_t (NULL = the legacy default stream, as the reference's
 *           `<<<grid, block, 0, 0>>>` launches use)
 *
 * Asynchronous like the reference: returns after the launch. Inputs are const
 * and are never written (the reference's pre-transpose path overwrites a and b,
 * 1-amd-fp8-mm/amd-fp8-mm-submission.py:152).
 */
int b200_fp8_mm(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c,
                int M, int N, int K,
                long long lda, long long ldb,
                long long sa_m, long long sa_k,
                long long sb_n, long long sb_k,
                long long ldc, int n_phase,
                void* workspace, size_t workspace_bytes,
                int* device_status, void* stream);

/* Same, with the plan given by the caller (block_n, cta_pair, split_k, stages,
 * store_bufs are read; 0 in any of them means "choose"; cta_pair -1 forces single
 * CTAs, store_bufs -1 forces plain stores). Used for sweeps and by the tests to
 * force every kernel variant. */
int b200_fp8_mm_planned(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c,
                        int M, int N, int K,
                        long long lda, long long ldb,
                        long long sa_m, long long sa_k,
                        long long sb_n, long long sb_k,
                        long long ldc, int n_phase,
                        void* workspace, size_t workspace_bytes,
                        int* device_status, void* stream,
                        const b200_fp8_mm_plan* forced);

/*
 * The same GEMM with both element strides of a and b given, so that either operand may be
 * stored MN-major: a as [K][M] (a_sm == 1, a_sk = bytes between consecutive k), b as [K][N]
 * (b_sn == 1). That is the storage the reference's kernels index (`a[k*m + i]`,
 * 1-amd-fp8-mm/amd-fp8-mm-submission.py:283-300) and the one its pre-transpose path
 * rewrites in place before the GEMM (same file, 128-154, 570-571); here the tile is loaded
 * as it lies and handed to the tensor core as an MN-major operand, nothing is transposed
 * or written.
 *
 *  a   element (i,kk) at a + i*a_sm + kk*a_sk; either a_sk == 1 (K-major, a_sm >= K) or
 *      a_sm == 1 (MN-major, a_sk >= M); the other stride a multiple of 16
 *  b   element (j,kk) at b + j*b_sn + kk*b_sk, same rule
 *  forced  NULL, or a plan as for b200_fp8_mm_planned. CTA pairs with an MN-major operand exist at
 *      block_n 192 and 256 for a, and at block_n 256 for b; forcing cta_pair = 1 elsewhere gives
 *      B200_FP8_MM_ERR_PLAN, and the automatic plan falls back to single CTAs there
 *
 * Everything else as for b200_fp8_mm. b200_fp8_mm_workspace_bytes covers both layouts.
 */
int b200_fp8_mm_strided(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c,
                        int M, int N, int K,
                        long long a_sm, long long a_sk,
                        long long b_sn, long long b_sk,
                        long long sa_m, long long sa_k,
                        long long sb_n, long long sb_k,
                        long long ldc, int n_phase,
                        void* workspace, size_t workspace_bytes,
                        int* device_status, void* stream,
                        const b200_fp8_mm_plan* forced);

/*
 * Grouped form: `groups` independent block-scaled GEMMs of the same N and K in one launch, for the
 * expert GEMMs of an MoE layer. (The reference's MoE submission runs its experts as fp16
 * `torch.bmm` calls, 2-amd-moe/amd-moe-submission.py:604-611; this is the FP8 block-scaled kernel
 * offered for that call site, one launch instead of one per expert.)
 *
 *  a        e4m3fn [groups][M][K],  element (g,i,kk) at a + g*a_g + i*lda + kk
 *  b        e4m3fn [groups][N][K],  element (g,j,kk) at b + g*b_g + j*ldb + kk
 *  a_scale  fp32, element (g,i,kb)  at a_scale + g*sa_g + i*sa_m + kb*sa_k
 *  b_scale  fp32, element (g,jb,kb) at b_scale + g*sb_g + jb*sb_n + kb*sb_k, jb = j/128
 *  c        bf16 [groups][M][N],    element (g,i,j) at c + g*c_g + i*ldc + j
 *  m_valid  NULL, or a DEVICE array int[groups]: only rows [0, m_valid[g]) of group g exist
 *           (clamped to [0, M]). Tiles past it are skipped, rows past it are not written. The
 *           array is read by the kernel, so it may be produced on the stream just before.
 *  lda, ldb, a_g, b_g multiples of 16; a and b 16-byte aligned; K a multiple of 128
 *  forced   NULL, or a plan (block_n, cta_pair, stages, store_bufs are read); every tile is whole:
 *           split_k > 1 gives B200_FP8_MM_ERR_PLAN. CTA pairs (256-row tiles inside each group)
 *           exist for block_n 192 and 256; they are chosen when M fills 256-row tiles to 7/8
 *
 * Needs no workspace. Asynchronous; inputs are never written.
 */
int b200_fp8_mm_grouped(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c,
                        int groups, int M, int N, int K,
                        long long lda, long long a_g,
                        long long ldb, long long b_g,
                        long long sa_g, long long sa_m, long long sa_k,
                        long long sb_g, long long sb_n, long long sb_k,
                        long long ldc, long long c_g,
                        const int* m_valid,
                        int* device_status, void* stream,
                        const b200_fp8_mm_plan* forced);

/*
 * The same GEMM for callers that cannot allocate device memory. (No counterpart in the
 * reference: its launcher gets its split-K scratch from torch.empty on every call.)
 *
 * Who needs it: code that is given input and output pointers and nothing else, and for which
 * cudaMalloc is not an option - an engine plug-in's enqueue hook, a latency-critical serving
 * loop that must not take the implicit device synchronisation of the allocator, a process
 * whose memory pools are frozen after start-up. b200_fp8_mm makes such a caller bring a
 * workspace for split-K plans; this entry point brings its own instead: a fixed 8 MiB array
 * inside the library's device image (b200_fp8_mm_static_scratch_limit() returns the size).
 * Every GPU that loads the library holds those 8 MiB until the process exits.
 *
 * Arguments as for b200_fp8_mm, without the workspace pair. It never calls cudaMalloc,
 * cudaFree or any allocating library routine. Problems whose plan needs more scratch than the
 * array holds are refused with B200_FP8_MM_ERR_SCRATCH_LIMIT (nothing is launched); plans that
 * do not split K need no scratch and always fit.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 * with that device current) and keeps it; make that first call outside any stream capture.
 * All calls share the one array, which keeps what the previous call left in it: once every
 * argument check has passed, the entry point zeroes the tile counters on `stream` right before
 * a launch that uses them (a refused call puts nothing on the stream), and two calls
 * that can overlap on the GPU (different streams, no dependency) would race on it - serialise
 * them, or use b200_fp8_mm with separate workspaces.
 */
int b200_fp8_mm_static_scratch(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c,
                               int M, int N, int K,
                               long long lda, long long ldb,
                               long long sa_m, long long sa_k,
                               long long sb_n, long long sb_k,
                               long long ldc, int n_phase,
                               int* device_status, void* stream);

/*
 * Self-test of the bounded waits (diagnostics; no counterpart in the reference, whose kernels
 * have no waits to bound). Runs the plain 64-wide single-CTA kernel on the given problem with
 * every mbarrier wait limited to wait_limit_ns (1 ms .. 100 ms) and with the copy of K block
 * `skip_kblock` of the first tile left out, so the waits that depend on that block run out.
 * The kernel returns by itself; device_status (required) then reads
 * {B200_FP8_MM_DEV_WAIT_EXPIRED, role/barrier, block, phase}, c is not valid, and the context
 * stays usable. Nothing traps and no wait is unbounded. Arguments a .. ldc as for b200_fp8_mm.
 */
int b200_fp8_mm_selftest_wait_expiry(const void* a, const void* b, const float* a_scale, const float* b_scale,
                                     void* c, int M, int N, int K,
                                     long long lda, long long ldb,
                                     long long sa_m, long long sa_k,
                                     long long sb_n, long long sb_k,
                                     long long ldc,
                                     unsigned long long wait_limit_ns, int skip_kblock,
                                     int* device_status, void* stream);

/* Size in bytes of the scratch array b200_fp8_mm_static_scratch uses. */
size_t b200_fp8_mm_static_scratch_limit(void);

/* Workspace the plan chosen by b200_fp8_mm / b200_fp8_mm_strided for (M,N,K) needs, in bytes
 * (0 when it does not split K; the larger of the two when the layouts' plans differ). The plan
 * depends on the SM count: the size is for the current CUDA device when there is one (the device
 * the GEMM will run on must be current), else for B200's 148 SMs. Replaces
 * the reference's per-call `torch.empty(m*n*4)` split-K scratch
 * (1-amd-fp8-mm/amd-fp8-mm-submission.py:597-601). */
size_t b200_fp8_mm_workspace_bytes(int M, int N, int K);

/* Workspace a forced plan needs (0 fields in *forced mean "choose"), rounded up to 256. */
size_t b200_fp8_mm_plan_workspace_bytes(int M, int N, int K, const b200_fp8_mm_plan* forced);

/* Fills *out with the plan b200_fp8_mm would use for this problem on a GPU with
 * sm_count SMs (0 = 148). Pure host arithmetic; needs no GPU. */
int b200_fp8_mm_describe(int M, int N, int K, int n_phase, int sm_count, b200_fp8_mm_plan* out);

/* The selector's own cost estimate for the plan it would pick, in SM clocks (about 1.9 GHz);
 * negative for a bad shape. Pure host arithmetic. Used to compare ways of cutting one problem into
 * per-GPU pieces; it is a model fitted to measurements, good to a few percent, not a promise. */
double b200_fp8_mm_estimate_clocks(int M, int N, int K, int sm_count);

/* Text for a return code. */
const char* b200_fp8_mm_strerror(int code);

/* Library version, bumped when the ABI changes. */
int b200_fp8_mm_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_FP8_MM_H_ */
