/*
 * mamba_b200 -- C ABI of the B200 (sm_100a) scan library, libmamba_b200.so.
 *
 * Three forward operators of state-spaces/mamba are served:
 *   Mamba-1 selective scan, the Mamba-2 SSD chunked scan, and the single-token
 *   decode state update.  The library never allocates or frees device memory,
 *   keeps no pointer after a call returns, never synchronises the device and
 *   never throws: every entry returns 0 or a negative MB200_ERR_* code and
 *   mb200_last_error() gives the text for the calling thread.  All kernels are
 *   enqueued on the cudaStream_t passed as `stream` (as a void*), on the device
 *   named by args->device (made current for the call).
 *
 * All strides are in ELEMENTS of the tensor they describe.  A stride of 0 is a
 * broadcast.  Optional tensors are NULL when absent.
 */
#ifndef MAMBA_B200_H
#define MAMBA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB200_OK               0
#define MB200_ERR_BAD_ARG     -1   /* a shape, stride, alignment or pointer the call cannot accept   */
#define MB200_ERR_UNSUPPORTED -2   /* a documented feature of the operator that this build lacks      */
#define MB200_ERR_LAUNCH      -3   /* the CUDA runtime refused a launch or an attribute change        */
#define MB200_ERR_NO_DEVICE   -4   /* no sm_100 device / wrong device index                           */

typedef enum mb200_dtype { MB200_F32 = 0, MB200_F16 = 1, MB200_BF16 = 2 } mb200_dtype;

/* Library version (major*10000 + minor*100 + patch) and last error text of this thread. */
int mb200_version(void);
const char *mb200_last_error(void);

/* ---------------------------------------------------------------------------------------------
 * Mamba-1 selective scan forward.
 * Replaces selective_scan_cuda.fwd (csrc/selective_scan/selective_scan.cpp:226-336, bound at
 * :494-497; kernel csrc/selective_scan/selective_scan_fwd_kernel.cuh:72-308), which
 * SelectiveScanFn.forward calls (mamba_ssm/ops/selective_scan_interface.py:58).
 *
 *   h_t = exp(dt_t A) h_{t-1} + dt_t B_t u_t ;  y_t = C_t . h_t + D u_t ;  out_t = y_t * silu(z_t)
 *   dt_t = delta_t + delta_bias, passed through softplus (identity above 20) when delta_softplus.
 *
 * u, delta, z, out, out_pregate : (batch, dim, seqlen), io_dtype, seqlen stride 1.
 * A : (dim, dstate) fp32.   D, delta_bias : (dim) fp32, contiguous.
 * B, C : when *_variable, (batch, ngroups, dstate, seqlen) io_dtype with seqlen stride 1 and
 *        strides {batch, group, dstate}; otherwise (dim, dstate) fp32 with strides {dim, dstate, 0}.
 * out        : gated output when z is given, else y.  out_pregate (optional, only with z): y.
 * last_state : optional (batch, dim, dstate) fp32 contiguous, h after the last step.
 * dstate <= 256.  Complex A is not supported (MB200_ERR_UNSUPPORTED is the caller's to raise).
 */
typedef struct mb200_scan_args {
    const void *u, *delta;
    const float *A;
    const void *B, *C;
    const float *D;
    const void *z;
    const float *delta_bias;
    void *out, *out_pregate;
    float *last_state;
    int32_t batch, dim, seqlen, dstate, ngroups;
    int32_t io_dtype;                 /* mb200_dtype of u, delta, z, out and of variable B, C */
    int32_t B_variable, C_variable, delta_softplus;
    int32_t device;
    int64_t u_stride[2], delta_stride[2], z_stride[2], out_stride[2], pregate_stride[2]; /* {batch, dim} */
    int64_t A_stride[2];              /* {dim, dstate} */
    int64_t B_stride[3], C_stride[3];
    void *scratch;                    /* optional, 16-byte aligned, see mb200_scan_scratch_bytes; NULL = none */
    size_t scratch_bytes;
} mb200_scan_args;

int mb200_selective_scan_fwd(const mb200_scan_args *args, void *stream);

/* No counterpart in the reference (its kernel walks a sequence from end to end inside one CTA,
 * csrc/selective_scan/selective_scan_fwd_kernel.cuh:102-103).  A call with few (batch, channel) rows -- one batch
 * row of a batch that was divided over several GPUs, say -- leaves most of the GPU idle if every row is walked from
 * end to end.  Lent a scratch buffer, the library cuts the sequence into segments that run side by side: a first
 * launch summarises each segment (end state from zero, product of decays), a fold chains the summaries, a second
 * launch runs every segment from its true entering state.  *bytes receives the size that enables this for the sizes
 * in args (pointers are not read), or 0 when the one-pass kernel is the faster choice.  Results agree with the
 * one-pass scan to fp32 rounding. */
int mb200_scan_scratch_bytes(const mb200_scan_args *args, size_t *bytes);

/* ---------------------------------------------------------------------------------------------
 * Mamba-1 selective scan, backward.
 * Replaces selective_scan_cuda.bwd (csrc/selective_scan/selective_scan.cpp:338-492, kernel
 * selective_scan_bwd_kernel.cuh), called at mamba_ssm/ops/selective_scan_interface.py:83-86.
 *
 * Inputs as in mb200_scan_args plus dout (batch, dim, seqlen) io_dtype = dL/d(out), where out is the gated
 * output when z is given.  The scan is recomputed from the inputs: neither the forward's prefix tensor `x` nor its
 * pre-gate output is read (the reference needs both, selective_scan_bwd_kernel.cuh:140-142,180-188).
 *
 * Outputs.  du, ddelta (and dz with z): (batch, dim, seqlen) io_dtype, last stride 1.  dA: (dim, dstate) fp32
 * contiguous.  dB, dC: fp32 contiguous in the shape of B, C -- (batch, ngroups, dstate, seqlen) when
 * input-dependent (the reference accumulates them in fp32 too, selective_scan.cpp:461-462, and casts afterwards),
 * (dim, dstate) otherwise.  dD, ddelta_bias: (dim) fp32, optional (NULL when D / delta_bias is NULL).
 * The library zeroes dA, dB, dC, dD, ddelta_bias on the stream before it accumulates into them.
 * The gradient with respect to last_state is not taken, as in the reference (selective_scan_interface.py:121-122).
 *
 * scratch: required, 16-byte aligned: the states at every eighth step (written by a first forward launch, read by the
 * backward launch that walks the sequence from the end) and, above 16 states, fp32 partial sums of du, ddelta, dz
 * between the passes over 16 states each.  mb200_scan_bwd_scratch_bytes() returns the size for the whole batch up to
 * 1 GiB; a larger batch is walked in slices of as many rows as the lent scratch holds (one row is the minimum).
 */
typedef struct mb200_scan_bwd_args {
    const void *u, *delta;
    const float *A;
    const void *B, *C;
    const float *D;
    const void *z;
    const float *delta_bias;
    const void *dout;
    void *du, *ddelta, *dz;
    float *dA, *dB, *dC, *dD, *ddelta_bias;
    int32_t batch, dim, seqlen, dstate, ngroups;
    int32_t io_dtype;                 /* mb200_dtype of u, delta, z, dout, du, ddelta, dz and of variable B, C */
    int32_t B_variable, C_variable, delta_softplus;
    int32_t device;
    int64_t u_stride[2], delta_stride[2], z_stride[2], dout_stride[2];    /* {batch, dim} */
    int64_t du_stride[2], ddelta_stride[2], dz_stride[2];
    int64_t A_stride[2];              /* {dim, dstate} */
    int64_t B_stride[3], C_stride[3]; /* as in mb200_scan_args */
    void *scratch;
    size_t scratch_bytes;
} mb200_scan_bwd_args;

int mb200_scan_bwd_scratch_bytes(const mb200_scan_bwd_args *args, size_t *bytes);
int mb200_selective_scan_bwd(const mb200_scan_bwd_args *args, void *stream);

/* Diagnostic, no counterpart in the reference.  The TMA-fed scan kernel bounds every wait on a copy or on
 * another warp; when a wait runs out it stops and records a non-zero code in a per-device word instead of
 * hanging.  This call copies that word to *status (0 = no wait has ever run out on `device`).  It
 * synchronises with the device, so it belongs in tests and post-mortems, not on the hot path. */
int mb200_scan_status(int device, int *status);

/* ---------------------------------------------------------------------------------------------
 * Single-token decode state update, state modified in place.
 * Replaces the launch in selective_state_update (mamba_ssm/ops/triton/selective_state_update.py:
 * 135-221, kernel :23-132).
 *
 *   dt = dt + dt_bias (softplus, identity above 20);  state <- state * exp(A dt) + (B dt) x
 *   out = sum_n state C + D x, then * silu(z)
 *
 * state : (nstates, nheads, dim, dstate) state_dtype.   x, z, out : (batch, nheads, dim) x_dtype.
 * dt : (batch, nheads, dim) dt_dtype.   A : (nheads, dim, dstate) fp32.
 * B, C : (batch, ngroups, dstate) bc_dtype.   D, dt_bias : (nheads, dim) fp32.
 * state_batch_indices : optional int32 (batch); row b uses state[idx[b]]; idx < 0 marks padding
 *   (out row written as 0, no state touched).
 * The call is a pure enqueue (no allocation, no host state), so it can sit inside a CUDA graph,
 * as the reference's generation loop requires (mamba_ssm/utils/generation.py:342-389).
 */
typedef struct mb200_ssu_args {
    void *state;
    const void *x, *dt;
    const float *A;
    const void *B, *C;
    const float *D;
    const void *z;
    const float *dt_bias;
    void *out;
    const int32_t *state_batch_indices;
    int32_t batch, nheads, dim, dstate, ngroups;
    int32_t state_dtype, x_dtype, dt_dtype, bc_dtype;
    int32_t dt_softplus;
    int32_t device;
    int64_t state_stride[4];          /* {batch, head, dim, dstate} */
    int64_t x_stride[3], dt_stride[3], z_stride[3], out_stride[3];   /* {batch, head, dim} */
    int64_t A_stride[3];              /* {head, dim, dstate} */
    int64_t B_stride[3], C_stride[3]; /* {batch, group, dstate} */
    int64_t D_stride[2], dt_bias_stride[2];                          /* {head, dim} */
} mb200_ssu_args;

int mb200_selective_state_update(const mb200_ssu_args *args, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Mamba-2 SSD chunked scan forward.
 * Replaces the five launches of _mamba_chunk_scan_combined_fwd
 * (mamba_ssm/ops/triton/ssd_combined.py:343-394): _chunk_cumsum_fwd (ssd_chunk_state.py:718-741),
 * _chunk_state_fwd (:812-842), _state_passing_fwd (ssd_state_passing.py:196-224),
 * _bmm_chunk_fwd (ssd_bmm.py:165-210) and _chunk_scan_fwd (ssd_chunk_scan.py:1259-1308).
 *
 * x, z, out : (batch, seqlen, nheads, headdim) io_dtype, headdim stride 1, strides {batch, seq, head}.
 * dt : (batch, seqlen, nheads) dt_dtype, strides {batch, seq, head}.   A, dt_bias : (nheads) fp32.
 * B, C : (batch, seqlen, ngroups, dstate) io_dtype, dstate stride 1, strides {batch, seq, group}.
 * D : (nheads) fp32, or (nheads, headdim) fp32 contiguous when D_has_hdim.
 * seq_idx : optional int32 (batch, seqlen) contiguous, non-decreasing sequence ids starting at 0 for packed
 *   sequences: positions with different ids do not interact (ssd_chunk_state.py:246-251, ssd_state_passing.py:76-79,
 *   ssd_bmm.py:84-88, ssd_chunk_scan.py:97-113).
 * cu_seqlens / num_seqs / varlen_states : optional (batch must be 1): int32 (num_seqs + 1) cumulative sequence
 *   lengths and an fp32 (num_seqs, nheads, headdim, dstate) output receiving the state after the last token of
 *   every packed sequence (chunk_state_varlen, ssd_chunk_state.py:1018-1044, kernel :639-715).
 * initial_states : optional (batch, nheads, headdim, dstate) fp32 contiguous.
 * final_states   : optional (batch, nheads, headdim, dstate) fp32 contiguous.
 * scratch : caller-owned device buffer of at least mb200_ssd_scratch_bytes() bytes, 256-byte
 *   aligned; holds dt, the dt*A cumulative sums, the per-chunk states and C.B^T between stages.  Its
 *   last 256 bytes hold an int32 status word, cleared at the start of every call: 0 after a clean run,
 *   non-zero if a kernel abandoned one of its bounded waits (the outputs of that call are then invalid).
 * phases : MB200_SSD_PHASE_ALL for the operator.  A sequence that is split across devices runs
 *   MB200_SSD_PHASE_LOCAL first (cumulative sums, per-chunk states, and -- with zero incoming state --
 *   the state at the end of the local range into final_states plus the product of the chunk decays
 *   into range_decay), exchanges states, then MB200_SSD_PHASE_OUTPUT with initial_states set to the
 *   incoming state (inter-chunk recurrence and chunk outputs; scratch must be untouched in between).
 *   C.B^T needs nothing from the exchange: a LOCAL call with MB200_SSD_PHASE_CB added (and C given) computes it as
 *   well, ahead of the exchange, and the OUTPUT call is then told so with MB200_SSD_PHASE_CB_READY.
 * range_decay : optional (batch, nheads) fp32, written in the LOCAL phase.
 */
#define MB200_SSD_PHASE_LOCAL    1
#define MB200_SSD_PHASE_OUTPUT   2
#define MB200_SSD_PHASE_ALL      3
#define MB200_SSD_PHASE_CB       4   /* with LOCAL alone: also form C.B^T in the scratch                    */
#define MB200_SSD_PHASE_CB_READY 8   /* with OUTPUT alone: the scratch already holds C.B^T of these inputs */

typedef struct mb200_ssd_args {
    const void *x, *dt;
    const float *A;
    const void *B, *C;
    const float *D;
    const void *z;
    const float *dt_bias;
    const int32_t *seq_idx;
    const float *initial_states;
    void *out;
    float *final_states;
    float *range_decay;
    void *scratch;
    size_t scratch_bytes;
    int32_t batch, seqlen, nheads, headdim, ngroups, dstate, chunk_size;
    int32_t io_dtype, dt_dtype;
    int32_t dt_softplus, D_has_hdim;
    float dt_min, dt_max;             /* clamp applied after softplus; {0, +inf} disables it */
    int32_t phases;
    int32_t device;
    int64_t x_stride[3], z_stride[3], out_stride[3], dt_stride[3], B_stride[3], C_stride[3];
    const int32_t *cu_seqlens;
    float *varlen_states;
    int32_t num_seqs;
    int32_t reserved_;
} mb200_ssd_args;

int mb200_ssd_scratch_bytes(const mb200_ssd_args *args, size_t *bytes);
int mb200_ssd_chunk_scan_fwd(const mb200_ssd_args *args, void *stream);

/*
 * SSD chunked scan for callers that cannot allocate device memory.
 * No counterpart in the reference (its operator allocates its intermediates through PyTorch on every call,
 * mamba_ssm/ops/triton/ssd_combined.py:374-387).
 *
 * Same operator and same argument struct as mb200_ssd_chunk_scan_fwd, but args->scratch and
 * args->scratch_bytes are ignored: the intermediates live in a buffer of MB200_SSD_STATIC_SCRATCH_BYTES
 * that is part of the library image, so every device that loads the library carries it until the process
 * exits.  It is meant for code that runs where allocation is off the table -- a plugin whose host framework
 * hands it a fixed memory plan, an enqueue callback that must not touch the allocator, a process whose
 * memory pool is already fully committed -- and only needs modest problem sizes.  A problem whose
 * mb200_ssd_scratch_bytes() exceeds the buffer is refused with MB200_ERR_BAD_ARG; nothing is launched.
 * The call performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * The first call on each device looks up the buffer's device address (one cudaGetSymbolAddress with that
 * device current); make that first call outside any stream capture.  All calls on a device share the one
 * buffer: it still holds the previous call's intermediates (the status word is cleared at the start of every
 * call, nothing else needs to start from zero), and two calls whose kernels overlap on the GPU -- different
 * streams, or different host threads -- race on it.  Serialise them.
 */
#define MB200_SSD_STATIC_SCRATCH_BYTES (32u << 20)
int mb200_ssd_chunk_scan_fwd_static(const mb200_ssd_args *args, void *stream);

/* Diagnostic for the call above, no counterpart in the reference: copies the status word that the last
 * mb200_ssd_chunk_scan_fwd_static call with these sizes left in the built-in buffer to *status (0 = every kernel ran
 * to completion).  Synchronises with the device; for tests and post-mortems, not for the hot path.  Callers of
 * mb200_ssd_chunk_scan_fwd read the word from their own scratch buffer (its last 256 bytes) instead. */
int mb200_ssd_static_status(const mb200_ssd_args *args, int *status);

/*
 * Folds an incoming state through a device's local range when a sequence is split across devices:
 *   s_out = range_decay[b,h] * s_in + s_local      over (batch*nheads) rows of `row` fp32 elements.
 * No counterpart in the reference (its SSD scan always sees the whole sequence on one device,
 * mamba_ssm/ops/triton/ssd_state_passing.py:72-80 being the recurrence this applies range-wise).
 * s_in may be NULL (treated as zero); s_out may alias s_local.
 */
int mb200_ssd_fold_state(const float *s_in, const float *range_decay, const float *s_local, float *s_out,
                         int64_t rows, int64_t row, int32_t device, void *stream);

/*
 * The same for a run of consecutive ranges in one launch (the all-gather hand-off: a rank folds the summaries of
 * all its predecessors).  `summaries` holds one record per range, `record_stride` floats apart: rows*row floats of
 * state followed by rows floats of decay.  Computes, in this order and with the arithmetic of
 * mb200_ssd_fold_state,   s = state[first];  for r = first+1 .. last:  s = decay[r] * s + state[r];   s_out = s.
 */
int mb200_ssd_fold_ranges(const float *summaries, int64_t record_stride, int32_t first, int32_t last, float *s_out,
                          int64_t rows, int64_t row, int32_t device, void *stream);

/* ---------------------------------------------------------------------------------------------
 * The element-wise steps either side of the scan inside the Mamba mixers.
 *
 * Causal depthwise conv1d, optionally followed by SiLU.  Replaces causal_conv1d_fn of the causal-conv1d package
 * (a dependency the reference does not vendor) as the mixers call it -- mamba_ssm/modules/mamba2.py:236-242,
 * mamba_ssm/modules/mamba_simple.py:172-177 -- whose CPU form is the depthwise nn.Conv1d with left padding at
 * mamba2.py:232-234:   out[b,c,t] = act(bias[c] + sum_k weight[c,k] * x[b,c,t - (width-1) + k]),  x = 0 before the start.
 *
 * x, out : (batch, dim, seqlen) io_dtype with strides {batch, dim, seq}; either layout (time or channels contiguous).
 * weight : (dim, width) contiguous, bias : optional (dim), both w_dtype.  width 2..4.
 * seq_idx : optional int32 (batch, seqlen) contiguous: taps that reach into another packed sequence read zero.
 * initial_states : optional (batch, dim, width-1) io_dtype, the inputs before t = 0.
 * final_states   : optional (batch, dim, width-1) io_dtype, receives the last width-1 inputs (the decode conv state).
 */
typedef struct mb200_conv1d_args {
    const void *x, *weight, *bias;
    const int32_t *seq_idx;
    const void *initial_states;
    void *final_states;
    void *out;
    int32_t batch, dim, seqlen, width;
    int32_t io_dtype, w_dtype;
    int32_t activation;               /* 0 none, 1 silu */
    int32_t device;
    int64_t x_stride[3], out_stride[3], init_stride[3], final_stride[3];
} mb200_conv1d_args;

int mb200_causal_conv1d_fwd(const mb200_conv1d_args *args, void *stream);

/* Single-token form (causal_conv1d_update of the same package; the reference's own code for it is the roll /
 * multiply / sum at mamba_ssm/modules/mamba2.py:309-315).  conv_state (batch, dim, state_len >= width-1) is shifted
 * left by one and x appended, in place; out[b,c] = act(bias[c] + sum_k weight[c,k] * window[k]) over the last width-1
 * old entries followed by x.  x, out : (batch, dim) io_dtype with strides {batch, dim}. */
typedef struct mb200_conv1d_update_args {
    const void *x, *weight, *bias;
    void *conv_state;
    void *out;
    int32_t batch, dim, width, state_len;
    int32_t io_dtype, w_dtype;
    int32_t activation;
    int32_t device;
    int64_t x_stride[2], out_stride[2], state_stride[3];
} mb200_conv1d_update_args;

int mb200_causal_conv1d_update(const mb200_conv1d_update_args *args, void *stream);

/* Gated RMSNorm after the SSD scan.  Replaces the launch in rmsnorm_fn / RMSNorm.forward
 * (mamba_ssm/ops/triton/layernorm_gated.py:415-437; definition rms_norm_ref :18-41), used at
 * mamba_ssm/modules/mamba2.py:269-270, 338-339:
 *   norm_before_gate = 1 :  out = x * rstd * weight (+ bias), then * silu(z)
 *   norm_before_gate = 0 :  x <- x * silu(z) first, then out = x * rstd * weight (+ bias)
 * with rstd = 1 / sqrt(mean(x^2) + eps) taken over each group of group_size consecutive columns.
 * x, z, out : (nrows, ncols) io_dtype, unit column stride, row strides given; weight, bias : (ncols) w_dtype. */
typedef struct mb200_rmsnorm_args {
    const void *x, *z, *weight, *bias;
    void *out;
    int64_t nrows;
    int32_t ncols, group_size;
    int32_t io_dtype, w_dtype;
    int32_t norm_before_gate;
    float eps;
    int32_t device;
    int32_t reserved_;
    int64_t x_stride, z_stride, out_stride;
} mb200_rmsnorm_args;

int mb200_rmsnorm_gated_fwd(const mb200_rmsnorm_args *args, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MAMBA_B200_H */
