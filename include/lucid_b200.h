/*
 * lucid_b200 -- C ABI of the B200 (sm_100a) quantized-inference kernels.
 *
 * Drop-in boundary for Lucid's quantization hot path.  Every entry point takes
 * plain device pointers and sizes; the caller owns all memory (inputs, outputs
 * and workspaces); nothing is retained after the call returns.  All work is
 * enqueued on the given CUDA stream (a cudaStream_t passed as void*; NULL is
 * the legacy default stream) and the functions return without synchronising.
 *
 * Return value: 0 on success, otherwise one of the LQ_ERR_* codes; the text of
 * the last failure on the calling thread is available from lq_last_error().
 * Codes map onto the reference's error taxonomy (lucid/_C/core/Error.h:63-495):
 * SHAPE -> ShapeMismatch, DTYPE -> DtypeMismatch, DEVICE -> DeviceMismatch,
 * UNSUPPORTED -> NotImplementedError, others -> LucidError.
 *
 * Arithmetic contract (bit-exact with the reference's CPU path): every step is
 * one IEEE binary32 operation in the reference's order, division is a true
 * divide, rounding is ties-to-even.
 */
#ifndef LUCID_B200_H_
#define LUCID_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LQ_VERSION 100

enum lq_status {
  LQ_OK = 0,
  LQ_ERR_SHAPE = 1,        /* sizes inconsistent or zero where not allowed            */
  LQ_ERR_DTYPE = 2,        /* dtype code not valid for this argument                  */
  LQ_ERR_DEVICE = 3,       /* null pointer where a device pointer is required         */
  LQ_ERR_ALIGNMENT = 4,    /* pointer / leading dimension violates a stated alignment */
  LQ_ERR_UNSUPPORTED = 5,  /* valid request this build does not implement             */
  LQ_ERR_WORKSPACE = 6,    /* workspace too small                                     */
  LQ_ERR_CUDA = 7,         /* CUDA runtime / driver error (text in lq_last_error)     */
  LQ_ERR_TIMEOUT = 8       /* a bounded device-side wait ran out                      */
};

enum lq_dtype {
  LQ_F32 = 0,
  LQ_BF16 = 1,
  LQ_S8 = 2,
  LQ_U8 = 3,
  LQ_S16 = 4, /* storage of the reference's quint8 codes (lucid/quantization/_qscheme.py:243) */
  LQ_S32 = 5
};

/* How scale / zero_point broadcast over a (rows, cols) view. */
enum lq_ch_mode {
  LQ_PER_TENSOR = 0, /* one value                                             */
  LQ_PER_ROW = 1,    /* one value per row    (ch_axis = 0; per-token)         */
  LQ_PER_COL = 2     /* one value per column (ch_axis = last)                 */
};

int lq_version(void);
/* Copies the calling thread's last error text (NUL terminated) into buf. */
int lq_last_error(char* buf, size_t n);

/* The library reads its LQ_* environment knobs (LQ_GEMM_SHAPE, LQ_GEMM_EPI_WARPS,
 * LQ_GEMM_STREAMK, LQ_GEMM_VERBOSE: force a tile shape / epilogue width / schedule of the
 * contraction, all numerically identical) once, at first use; this re-reads them (tests switch
 * variants inside one process). */
void lq_reload_env(void);

/* ---- calibration ------------------------------------------------------- */

/* Bytes of workspace lq_minmax needs for the per-tensor mode.  The workspace
 * must be zero-filled once before its first use; the kernel leaves it zeroed
 * again, so it can be reused by later calls on the same stream. */
size_t lq_minmax_workspace_bytes(void);

/* Number of launches of the bulk-copy pipelined stream kernels (dequantize, per-token encode of
 * long rows) on the current device that gave up on a bounded wait since the last call; the
 * count is cleared.  Such a launch left its output incomplete.  Synchronises the device. */
int lq_stream_timeouts(unsigned int* count);

/* Running-range reduction.
 * Replaces MinMaxObserver.forward (lucid/quantization/observer.py:364-370; the
 * x.min()/x.max() pair of lucid/nn/quantized/dynamic/linear.py:87-89) for
 * mode = LQ_PER_TENSOR and PerChannelMinMaxObserver.forward
 * (lucid/quantization/observer.py:635-648) for mode = LQ_PER_ROW.
 * x: (rows, cols) row-major, in_dtype LQ_F32 or LQ_BF16.
 * out_min / out_max: 1 float (per tensor) or rows floats. */
int lq_minmax(const void* x, int in_dtype, size_t rows, size_t cols, int mode, float* out_min,
              float* out_max, void* workspace, size_t workspace_bytes, void* stream);

/* Per-tensor range reduction that allocates nothing and takes no workspace.
 * (No counterpart in the reference: it exists for callers of this library that
 * cannot allocate device memory where they need a range -- code inside an arena
 * or pool owner that forbids nested allocation, latency-critical threads that
 * must not touch an allocator, and foreign-language hosts that bind only this
 * header.)  The scratch that lq_minmax takes from its caller lives in a fixed
 * array of about 10 KB inside the library image; every GPU that loads the
 * library holds that array until the process exits.
 *
 * x: n contiguous elements (LQ_F32 | LQ_BF16); out_min / out_max: 1 float each.
 * n must not exceed lq_minmax_noalloc_max_elems() (2^30); larger inputs are
 * rejected with LQ_ERR_SHAPE -- use lq_minmax with a workspace for those.
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and caches it; make that
 * first call outside any stream capture.  All calls on a device share the one
 * array: the call re-arms it on `stream` before launching, so calls that are
 * ordered on a stream are safe, while calls that can overlap on the GPU
 * (different streams, different host threads) race and must be serialised by
 * the caller.  Results are identical to lq_minmax in per-tensor mode. */
size_t lq_minmax_noalloc_max_elems(void);
int lq_minmax_noalloc(const void* x, int in_dtype, size_t n, float* out_min, float* out_max,
                      void* stream);

/* Bytes of workspace lq_histc needs (zero-filled once before its first use; the kernel
 * leaves it zeroed again), and the largest bin count it accepts. */
size_t lq_histc_workspace_bytes(void);
int lq_histc_max_bins(void);

/* One batch of the histogram observer in one pass over x.
 * Replaces histc (lucid/_C/ops/composite/Stats.cpp:47-91; counting loop
 * lucid/_C/backend/cpu/CpuBackend.h:13276-13318) and, around it, what
 * HistogramObserver.forward does per batch (lucid/quantization/observer.py:819-838): the
 * x.min() / x.max() pair and the fold of the running histogram, re-binned onto the wider range
 * when the range grew (HistogramObserver._rebin, observer.py:786-817).
 *   counts[b] = #{ v in x : lo <= v <= hi, b = min(trunc((double(v) - lo) / ((hi - lo) / bins)), bins - 1) }
 *   hist_out  = float(counts)                                   prev_hist == NULL
 *             = float(counts) + prev_hist                       prev range == [lo, hi]
 *             = float(counts) + rebin(prev_hist onto [lo, hi])  otherwise
 * The bin index is the reference's binary64 expression bit for bit; NaN elements are skipped
 * (the reference's cast of NaN to an index is undefined).  lo < hi, both finite: a caller
 * with an empty range derives one from the data first, as the reference's histc does.
 * x: n contiguous elements (LQ_F32 | LQ_BF16).  hist_out: bins floats; it may be prev_hist.
 * out_min / out_max: optional (NULL to skip), 1 float each: the min / max of x from the same
 * pass, so a caller can bin against its current range and learn whether the range held. */
int lq_histc(const void* x, int in_dtype, size_t n, double lo, double hi, int bins,
             const float* prev_hist, double prev_lo, double prev_hi, float* hist_out,
             float* out_min, float* out_max, void* workspace, size_t workspace_bytes, void* stream);

/* One step of the histogram observer with its state on the device: two kernel launches, no
 * host synchronisation.  Replaces HistogramObserver.forward
 * (lucid/quantization/observer.py:819-838), which reads the batch's min / max and its own
 * range back to the host every batch.
 *   min_val, max_val: 1 float each, the running range; (+inf, -inf) before the first batch.
 *   hist:             bins floats, the running histogram.
 * The first kernel bins x on the current range while measuring x's own range; if the range
 * held, it folds the running histogram and the step is complete after one pass over x.
 * Otherwise (first batch, wider range, constant history) it stores the new range, and the
 * second kernel -- which returns at once when it is not needed -- bins x on the new range and
 * folds the running histogram, re-binned from the old range.  Results are those of lq_histc
 * driven by the reference's host logic, bit for bit.  A batch without a finite value leaves
 * the state unchanged.  Workspace: as lq_histc (the two may share one, in stream order). */
int lq_histogram_observe(const void* x, int in_dtype, size_t n, int bins, float* min_val,
                         float* max_val, float* hist, void* workspace, size_t workspace_bytes,
                         void* stream);

/* (scale, zero_point) from observed ranges, on device.
 * Replaces calculate_qparams (lucid/quantization/_qparams.py:190-215). */
int lq_calculate_qparams(const float* min_val, const float* max_val, size_t n, int symmetric,
                         int is_signed, int qmin, int qmax, float eps, float* scale,
                         float* zero_point, void* stream);

/* ---- affine encode / decode ------------------------------------------- */

/* q = clip(rint(x / s) + z, qmin, qmax) cast to out_dtype.
 * Replaces quantize (lucid/quantization/_functional.py:164-182).
 * scale / zero_point are device pointers (1, rows or cols floats according to
 * ch_mode); when scale is NULL the host scalars scale_value / zp_value are used
 * (ch_mode must be LQ_PER_TENSOR).  in_dtype LQ_F32 | LQ_BF16; out_dtype LQ_S8 |
 * LQ_U8 | LQ_S16. */
int lq_quantize(const void* x, int in_dtype, size_t rows, size_t cols, const float* scale,
                const float* zero_point, float scale_value, float zp_value, int ch_mode, int qmin,
                int qmax, void* out, int out_dtype, void* stream);

/* Dynamic per-tensor encode in one call: observed range -> (scale, zero_point) -> codes, all
 * on the device (no host round trip).  Replaces the x.min() / x.max() -> calculate_qparams ->
 * fake_quantize prologue of dynamic.Linear.forward (lucid/nn/quantized/dynamic/linear.py:87-92).
 * workspace as for lq_minmax; out_scale / out_zp: 1 float each; out_minmax: 2 floats. */
int lq_quantize_dynamic(const void* x, int in_dtype, size_t rows, size_t cols, int symmetric,
                        int is_signed, int qmin, int qmax, float eps, void* workspace,
                        size_t workspace_bytes, void* out, int out_dtype, float* out_scale,
                        float* out_zp, float* out_minmax, void* stream);

/* x = (f32(q) - z) * s.  Replaces dequantize
 * (lucid/quantization/_functional.py:269-281).  q_dtype LQ_S8 | LQ_U8 | LQ_S16;
 * out_dtype LQ_F32 | LQ_BF16 (bf16 = the f32 result rounded once). */
int lq_dequantize(const void* q, int q_dtype, size_t rows, size_t cols, const float* scale,
                  const float* zero_point, float scale_value, float zp_value, int ch_mode,
                  void* out, int out_dtype, void* stream);

/* (clip(rint(x / s) + z, qmin, qmax) - z) * s, forward only.  Replaces
 * _FakeQuantizeAffine.forward (lucid/quantization/_functional.py:299-313).
 * When mask is non-NULL the straight-through saturation mask
 * (lucid/quantization/_functional.py:315-317) is written as f32 0/1. */
int lq_fake_quantize(const float* x, size_t rows, size_t cols, const float* scale,
                     const float* zero_point, float scale_value, float zp_value, int ch_mode,
                     int qmin, int qmax, float* out, float* mask, void* stream);

/* Per-token symmetric activation encode in one pass over HBM: row abs-max ->
 * scale = max(absmax / ((qmax - qmin) / 2), eps) -> codes.  Equals
 * PerChannelMinMaxObserver(ch_axis=0) -> calculate_qparams(symmetric, signed)
 * -> quantize(ch_axis=0) (lucid/quantization/observer.py:635-648,
 * _qparams.py:203-207, _functional.py:180-182).  in_dtype LQ_F32 | LQ_BF16
 * (bf16 is upcast to f32 first).  out: int8 (rows, cols); out_scale: rows. */
int lq_quantize_per_token(const void* x, int in_dtype, size_t rows, size_t cols, int qmin, int qmax,
                          float eps, int8_t* out, float* out_scale, void* stream);

/* ---- contraction -------------------------------------------------------- */

enum lq_activation { LQ_ACT_NONE = 0, LQ_ACT_RELU = 1, LQ_ACT_SILU_GATE = 2 };

/* Epilogue applied to the exact int32 accumulator acc[m,n] = sum_k a[m,k]*b[n,k]:
 *
 *   t = acc - a_zp * b_rowsum[n]                       (exact, int32)
 *   out_dtype LQ_S32:  out = t
 *   otherwise:         y = f32(t) * (a_scale[m] * b_scale[n])
 *                      y = y + bias[n]                  (if bias)
 *                      y = max(y, 0)                    (LQ_ACT_RELU)
 *     LQ_F32 / LQ_BF16: out = y (bf16: rounded once)
 *     LQ_S8 / LQ_U8:    out = clip(rint(y / out_scale) + out_zp, qmin, qmax)
 *
 * Every float step is a separate binary32 operation (no FMA contraction).
 * LQ_ACT_SILU_GATE: b holds [gate; up] interleaved in blocks of 128 rows; the
 * output has N/2 columns: silu(y_gate) * y_up.
 *
 * This is the integer form of nn.quantized.Linear.forward
 * (lucid/nn/quantized/linear.py:199-215) and dynamic.Linear.forward
 * (lucid/nn/quantized/dynamic/linear.py:84-99), which the reference evaluates
 * as dequantize -> float GEMM -> fake_quantize. */
typedef struct lq_epilogue {
  int32_t out_dtype;       /* lq_dtype of out                                     */
  int32_t act;             /* lq_activation                                       */
  int32_t a_scale_mode;    /* LQ_PER_TENSOR (1 float) or LQ_PER_ROW (M floats)    */
  int32_t qmin, qmax;      /* requantisation grid (LQ_S8 / LQ_U8 outputs)         */
  int32_t reserved;
  const float* a_scale;    /* device                                              */
  const float* a_zp;       /* device, 1 float holding an integer value, or NULL   */
  const int32_t* b_rowsum; /* device, N ints: sum_k b[n,k]; required with a_zp    */
  const float* b_scale;    /* device, N floats                                    */
  const float* bias;       /* device, N floats, or NULL                           */
  const float* out_scale;  /* device, 1 float (requantising outputs)              */
  const float* out_zp;     /* device, 1 float                                     */
} lq_epilogue_t;

/* out(M, N) = epilogue(a(M, K) . b(N, K)^T); a and b are K-contiguous 8-bit
 * codes (a signed or unsigned, b signed); K % 16 == 0 and a, b 16-byte aligned
 * (TMA), ldo in elements of out.  Needs no workspace.
 * `status` (device, 1 int32, may be NULL) receives LQ_ERR_TIMEOUT if a bounded
 * device-side wait ran out; it is left untouched otherwise. */
int lq_gemm_s8(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
               const lq_epilogue_t* ep, void* out, size_t ldo, int32_t* status, void* stream);

/* Bytes of scratch lq_gemm_s8_ws / lq_gemm_s8_sharded / lq_conv2d_nhwc_s8_ex can use (about
 * 24 MB: one 128 x 256 int32 partial tile per SM plus a 4 KB header).  Zero-fill it once before
 * its first use; every launch leaves it zeroed again.  One workspace serves one stream at a time.
 * After a call reported LQ_ERR_TIMEOUT through its status word, zero the workspace again. */
size_t lq_gemm_workspace_bytes(void);

/* lq_gemm_s8 with a scratch workspace: when the tile count does not fill whole waves of SMs,
 * the k-blocks of all tiles are dealt out in equal contiguous runs ("stream-K") and tiles cut
 * by a run boundary are completed from int32 partial sums in the workspace (integer addition,
 * so the result is bit-identical to lq_gemm_s8).  workspace == NULL behaves as lq_gemm_s8. */
int lq_gemm_s8_ws(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
                  const lq_epilogue_t* ep, void* out, size_t ldo, void* workspace,
                  size_t workspace_bytes, int32_t* status, void* stream);

/* The same contraction with the exchange step of an output-channel-sharded Linear fused
 * into its epilogue: every finished tile is stored into ALL `n_dst` destinations (1..8), each
 * the base of a row-major (M, ldo) buffer, at column offset `col0`.  outs[0] is normally this
 * GPU's own buffer and outs[1..] the same buffer on its peers, mapped into this process
 * (CUDA IPC / symmetric memory); the stores are plain peer stores over NVLink and overlap the
 * mainloop of the following tiles, replacing an all-gather of (M, N) shards plus a re-layout.
 * `outs` is a HOST array of device pointers.  The caller orders consumers after the kernels of
 * all ranks (a barrier across the ranks on the stream).  No counterpart in the reference,
 * which has no distributed code. */
int lq_gemm_s8_bcast(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
                     const lq_epilogue_t* ep, void* const* outs, int n_dst, size_t ldo,
                     size_t col0, int32_t* status, void* stream);

/* Per-token symmetric int8 encode of a COLUMN SHARD with the exchange fused in: row r of
 * x (rows x cols, row stride ldx; LQ_F32 | LQ_BF16) is encoded with
 * scale[r] = max(absmax[r] / ((qmax - qmin) / 2), eps) -- the expressions of
 * lq_quantize_per_token -- and the codes are stored at columns [col0, col0 + cols) of every
 * one of the n_dst (1..8) row-major (rows, ldo) int8 destinations: this GPU's buffer and the
 * peers' copies mapped into this process (plain peer stores over NVLink; n_dst = -1: outs[0] is
 * the buffer's NVSwitch multicast address).  absmax[r] is the per-token max |x| over ALL shards:
 * the maximum of row_absmax[p * absmax_stride + r] over p < absmax_parts, one part per rank
 * (filled by lq_absmax_rows_bcast, or one part holding an all-reduced value; max is order-free,
 * so the scales and codes equal the single-GPU encode of the unsharded tensor bit for bit).
 * out_scale (optional): rows floats.  `outs` is a HOST array of device pointers.  No
 * counterpart in the reference, which has no distributed code. */
int lq_quantize_rows_bcast(const void* x, int in_dtype, size_t rows, size_t cols, size_t ldx,
                           const float* row_absmax, int absmax_parts, size_t absmax_stride,
                           int qmin, int qmax, float eps, void* const* outs, int n_dst, size_t ldo,
                           size_t col0, float* out_scale, void* stream);

/* Per-row max |x| of a column shard (rows x cols, row stride ldx), stored at
 * outs[k][slot0 + r] for each of the n_dst (1..8) float tables: the max all-reduce that the
 * sharded per-token encode needs, as plain peer stores (rank p passes slot0 = p * rows, and
 * lq_quantize_rows_bcast reads the table with absmax_parts = ranks).  No counterpart in the
 * reference. */
int lq_absmax_rows_bcast(const void* x, int in_dtype, size_t rows, size_t cols, size_t ldx,
                         float* const* outs, int n_dst, size_t slot0, void* stream);

/* lq_quantize_per_token of a ROW shard of a replicated activation with the exchange fused in:
 * this rank encodes its `rows` rows (cols % 16 == 0, contiguous) and stores the codes at rows
 * [row0, row0 + rows) of each of the n_dst (1..8) (total_rows, cols) int8 buffers in `outs` --
 * or once through multicast_out, the buffer's NVSwitch multicast address, when that is not
 * NULL -- and the scales at scale_outs[k][row0 + r].  Each rank thus encodes 1 / ranks of the
 * tokens instead of all of them.  No counterpart in the reference. */
int lq_quantize_per_token_bcast(const void* x, int in_dtype, size_t rows, size_t cols, int qmin, int qmax,
                                float eps, void* const* outs, float* const* scale_outs, int n_dst,
                                void* multicast_out, size_t row0, void* stream);

/* lq_gemm_s8_bcast through NVSwitch multicast: `multicast_out` is the multicast address of a
 * row-major (M, ldo) buffer that every rank of the group has bound (CUDA multicast object /
 * torch symmetric memory `multicast_ptr`).  Each finished 16-byte piece is issued ONCE as a
 * multimem store and the switch writes it into every rank's buffer (this GPU's included), so a
 * GPU's egress is its own output volume instead of (ranks - 1) times it.  Rows, column offset
 * and output width must be multiples of 16 bytes.  Consumers are ordered after the kernels of
 * all ranks by the caller, as for lq_gemm_s8_bcast.  (lq_quantize_rows_bcast takes the same
 * kind of address with n_dst = -1.)  No counterpart in the reference. */
int lq_gemm_s8_multicast(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
                         const lq_epilogue_t* ep, void* multicast_out, size_t ldo, size_t col0,
                         int32_t* status, void* stream);

/* lq_gemm_s8_bcast / lq_gemm_s8_multicast plus the signal of the exchange step, so that no
 * collective has to follow the kernel: once every CTA has stored its tiles, the kernel adds 1 to
 * *signal_counter (a device word of this rank, zero before the first step) and stores the new
 * value, with release semantics at system scope, into each of the n_flags (<= 8) addresses in
 * `peer_flags` -- this rank's flag word on every rank that consumes the buffer (its own
 * included), e.g. element `rank` of a flags array in symmetric memory.  Consumers wait with
 * lq_peer_wait.  n_dst = 1..8: `outs` holds that many destinations (plain peer stores);
 * n_dst = -1: outs[0] is the buffer's NVSwitch multicast address.  `outs` and `peer_flags` are
 * HOST arrays of device pointers.  The workspace (lq_gemm_workspace_bytes) is required.  No
 * counterpart in the reference, which has no distributed code. */
int lq_gemm_s8_sharded(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
                       const lq_epilogue_t* ep, void* const* outs, int n_dst, size_t ldo, size_t col0,
                       int32_t* const* peer_flags, int n_flags, int32_t* signal_counter,
                       void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* Signal without a GEMM: a one-thread kernel that adds 1 to *signal_counter and stores the new
 * value (release, system scope) into the n_flags addresses; everything enqueued on `stream`
 * before it -- e.g. an encode kernel that stored into the peers' buffers -- has completed by then. */
int lq_peer_signal(int32_t* const* peer_flags, int n_flags, int32_t* signal_counter, void* stream);

/* Consumer side of the exchange: a one-warp kernel that adds 1 to *epoch (a device word of this
 * rank, zero before the first step) and waits until each of the n (<= 32) words flags[0..n) has
 * reached the new value (acquire loads at system scope; the producers count steps the same
 * way, so the comparison is "at least").  Work enqueued on `stream` after it sees every store
 * the producers made before their signals.  The wait is bounded: after timeout_cycles SM clock
 * cycles (0 = about one second) the kernel gives up, writes LQ_ERR_TIMEOUT to *status (optional)
 * and returns; nothing traps or spins forever. */
int lq_peer_wait(const int32_t* flags, int n, int32_t* epoch, long long timeout_cycles,
                 int32_t* status, void* stream);

/* sum_k b[n,k] for the zero-point correction term (N ints). */
int lq_rowsum_s8(const int8_t* b, size_t N, size_t K, int32_t* out, void* stream);

/* NHWC implicit-GEMM convolution on 8-bit codes with KRSC signed weights:
 * out[n,p,q,k] = epilogue(sum_{r,s,c} x[n, p*stride+r-pad, q*stride+s-pad, c] * w[k,r,s,c]).
 * Out-of-image taps read code 0, which is exact when the activation zero point
 * is 0 (symmetric or post-ReLU grids).  Integer form of
 * nn.quantized.Conv2d.forward (lucid/nn/quantized/conv.py:168-184).
 * C % 16 == 0; ep->a_zp must be NULL. */
int lq_conv2d_nhwc_s8(const void* x, int x_signed, const int8_t* w, size_t N, size_t H, size_t W,
                      size_t C, size_t K, size_t R, size_t S, size_t stride, size_t pad,
                      const lq_epilogue_t* ep, void* out, int32_t* status, void* stream);

/* General geometry of the NHWC convolution: what nn.quantized.Conv2d accepts
 * (lucid/nn/quantized/conv.py:119-184: stride, dilation, groups, explicit or "same" padding).
 * x: (N, H, W, C) codes; w: (K, R, S, C / groups) signed codes, the filters of group g at rows
 * [g*K/groups, (g+1)*K/groups); out: (N, P, Q, K).
 *   out[n,p,q,k] = epilogue(sum_{r,s,c} x[n, p*stride_h + r*dil_h - pad_h,
 *                                         q*stride_w + s*dil_w - pad_w, g(k)*C/groups + c] * w[k,r,s,c])
 * pad_h / pad_w are the padding BEFORE the first row / column; rows and columns past the far edge
 * read code 0 as well, so an asymmetric "same" padding is expressed by P and Q alone.
 * C / groups must be a multiple of 16. */
typedef struct lq_conv_geometry {
  size_t N, H, W, C;       /* input                                          */
  size_t K, R, S;          /* filters                                        */
  size_t P, Q;             /* output extent                                  */
  size_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w, groups;
} lq_conv_geometry_t;

/* lq_conv2d_nhwc_s8 for any stride (<= 8), dilation, group count and padding, with an optional
 * workspace as for lq_gemm_s8_ws (NULL: none).  One launch per group. */
int lq_conv2d_nhwc_s8_ex(const void* x, int x_signed, const int8_t* w, const lq_conv_geometry_t* geometry,
                         const lq_epilogue_t* ep, void* out, void* workspace, size_t workspace_bytes,
                         int32_t* status, void* stream);

/* ---- element-wise ops of the quantized region ----------------------------------------- */

enum lq_merge_op {
  LQ_MERGE_ADD = 0,      /* x + y        QFunctional.add / add_scalar                       */
  LQ_MERGE_MUL = 1,      /* x * y        QFunctional.mul / mul_scalar                       */
  LQ_MERGE_ADD_RELU = 2, /* relu(x + y)  QFunctional.add_relu                               */
  LQ_MERGE_COPY = 3      /* x            each piece of QFunctional.cat; a requantization    */
};

/* out = fake_quantize(op(x, y)) on the grid (out_scale, out_zp, qmin, qmax): the merges of
 * QFunctional (lucid/nn/quantized/functional_module.py:230-258), in one pass.
 * An operand is either values (LQ_F32 | LQ_BF16; scale / zero_point NULL) or codes
 * (LQ_S8 | LQ_U8 | LQ_S16 with its per-tensor device scale / zero_point), which are dequantized
 * in registers exactly as lq_dequantize would ((q - z) * s).  y == NULL selects the scalar
 * operand y_scalar.  The arithmetic is the reference's float32 sequence: op, relu, then
 * clip(rint(t / S) + Z).  Outputs, either or both: out_codes (codes_dtype LQ_S8 | LQ_U8 |
 * LQ_S16) and out_f32 = (code - Z) * S, the tensor the reference returns.  n elements. */
int lq_qmerge(int op, const void* x, int x_dtype, const float* x_scale, const float* x_zp,
              const void* y, int y_dtype, const float* y_scale, const float* y_zp, float y_scalar,
              size_t n, const float* out_scale, const float* out_zp, int qmin, int qmax,
              void* out_codes, int codes_dtype, float* out_f32, void* stream);

/* out[i] = table[in[i]] over n bytes; `table` is 256 bytes on the device.  The quantized
 * activations (lucid/nn/quantized/activation.py:22-60: float activation, then fake_quantize)
 * applied to 8-bit codes are a function of one byte, so the caller evaluates
 * encode(act(decode(c))) for the 256 codes once and streams the tensor through the table. */
int lq_lut_u8(const void* in_codes, size_t n, const uint8_t* table, void* out_codes, void* stream);

/* out[i] = table[x[i] * 256 + y[i]] over n byte pairs; `table` is 65536 bytes on the device
 * (16-byte aligned), held in shared memory by every CTA.  A QFunctional merge of two tensors of
 * 8-bit codes is a function of two bytes: the caller runs lq_qmerge once over the 65536 code
 * pairs of its grids and streams the tensors through the result, which is bit-identical to
 * lq_qmerge by construction and costs one shared load per element instead of an IEEE division.
 * out_f32 (optional): (code - out_zp) * out_scale, the code read as int8 when out_signed. */
int lq_lut2_u8(const void* x_codes, const void* y_codes, size_t n, const uint8_t* table,
               void* out_codes, float* out_f32, const float* out_scale, const float* out_zp,
               int out_signed, void* stream);

/* ---- recurrent cell -------------------------------------------------------------------- */

/* Pointwise part of one LSTM time step on the pre-activations gates (batch, 4 * hidden; row
 * stride ldg; gate order i, f, g, o):  c_out = sigmoid(f) * c_prev + sigmoid(i) * tanh(g),
 * h_out = sigmoid(o) * tanh(c_out); h_out has row stride ldh; c_out may alias c_prev.  Float32.
 * The weight-only quantized LSTM (lucid/nn/quantized/dynamic/rnn.py:67-87) runs the float cell
 * on dequantized weights; this replaces the element-wise passes of that cell with one kernel. */
int lq_lstm_cell_f32(const float* gates, size_t ldg, const float* c_prev, float* h_out, size_t ldh,
                     float* c_out, size_t batch, size_t hidden, void* stream);

/* ---- group-wise weight-only codes (4 / 8 bits) ------------------------------------------- */

/* The reference's low-precision weight route (lucid/quantization/_qgemm.py:69-152 `quantize`,
 * :155-225 `dequantize`, :228-320 `quantized_matmul`; engine ops
 * lucid/_C/ops/quantized/QuantizedMatmul.cpp:47-109): the input axis of a float32 (N, K) weight
 * is cut into groups of group_size (32 | 64 | 128) elements, each with
 * scale = (max - min) / (2^bits - 1) and bias = min (a constant group takes scale 1);
 * code = clip(rint((w - bias) / scale), 0, 2^bits - 1), bits = 4 | 8, packed little-endian into
 * 32-bit words: packed (N, K * bits / 32), scales / biases (N, K / group_size). */
int lq_groupwise_quantize(const float* w, size_t N, size_t K, int group_size, int bits, uint32_t* packed,
                          float* scales, float* biases, void* stream);
/* w_hat = code * scale + bias, float32 (N, K). */
int lq_groupwise_dequantize(const uint32_t* packed, const float* scales, const float* biases, size_t N,
                            size_t K, int group_size, int bits, float* out, void* stream);
/* out (M, N) = x (M, K) * w_hat^T (+ bias[N]) (ReLU when relu != 0), the weight decoded inside the
 * kernel; x and out share a dtype (LQ_F32 | LQ_BF16), float32 accumulation; row strides ldx / ldo
 * in elements; x rows and `packed` 16-byte aligned.  Built for decode shapes (a few activation
 * rows): the packed weight is streamed once per block of four rows. */
int lq_groupwise_matmul(const void* x, int x_dtype, size_t M, size_t ldx, const uint32_t* packed,
                        const float* scales, const float* biases, size_t N, size_t K, int group_size,
                        int bits, const float* bias, int relu, void* out, size_t ldo, void* stream);

/* ---- quantized embedding tables -------------------------------------------------------- */

/* Gather + dequantize of the rows of a per-row int8 table.  Replaces the forward of
 * nn.quantized.Embedding / EmbeddingBag (lucid/nn/quantized/sparse.py:141-146, 292-301), which
 * dequantize the whole table on every call before gathering; here only the rows asked for are
 * read.  weight: (num_embeddings, dim) codes; scale / zero_point: num_embeddings floats
 * (dequantize with ch_axis = 0).  indices: n_idx int32 (index_bits 32) or int64 (64).
 *   offsets == NULL: out[i, :] = dequantized row indices[i] (LQ_F32 | LQ_BF16); a row equal to
 *     padding_idx (pass -1 for none) is zeros, as in the engine's embedding_forward
 *     (lucid/_C/backend/cpu/CpuBackend.h:8970-9010).  An index outside the table leaves its row
 *     zero and writes LQ_ERR_SHAPE to *status (optional device word; the reference checks on
 *     the host).
 *   offsets != NULL: n_bags bag starts (same integer width as indices); out[b, :] (LQ_F32) pools
 *     bag b with mode 0 = sum, 1 = mean, 2 = max exactly as embedding_bag_forward
 *     (CpuBackend.h:5989-6080): rows added in index order, padding and out-of-range indices
 *     skipped, the mean divided by the number of rows added, an empty max bag = zeros. */
int lq_embedding_s8(const int8_t* weight, const float* scale, const float* zero_point,
                    size_t num_embeddings, size_t dim, const void* indices, int index_bits, size_t n_idx,
                    const void* offsets, size_t n_bags, int include_last_offset, int mode,
                    long long padding_idx, void* out, int out_dtype, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LUCID_B200_H_ */
