// Shared definitions of the SSD (Mamba-2) chunked forward: scratch layout and stage entry points.
#pragma once

#include "common.cuh"

namespace mb200 {

// Scratch the SSD stages hand to each other (all fp32, each region 256-byte aligned):
//   dt      (batch, nheads, nchunks, Q)        dt after bias/softplus/clamp, 0 past seqlen
//   dA_cum  (batch, nheads, nchunks, Q)        inclusive cumsum of dt*A inside each chunk
//   states  (batch, nchunks, nheads, P, N)     chunk states; the inter-chunk recurrence then
//                                              overwrites slot c with the state ENTERING chunk c
//   cb      (batch, nchunks, ngroups, Q, Q)    C.B^T per chunk (lower block triangle only); fp32 for the
//                                              general kernels, 16-bit in the same region for the tensor-core ones
//   prev16  (batch, nchunks, nheads, P, N)     16-bit copy of the state entering each chunk (tensor-core path);
//                                              (.., N, P) when the fused state-stream kernel wrote it
//   aux     sequence-split hand-over of the fused state-stream path, written by the LOCAL phase for the OUTPUT
//           phase: prefix decay (batch, nheads, nchunks), the range's end state from a zero incoming state
//           (batch, nheads, P, N) and the range decay (batch, nheads), all fp32
//   seq     packed sequences on the tensor-core path: for every position the offset inside its chunk at which its
//           sequence starts (batch, nchunks, Q) uint8, and per chunk whether its first position continues the
//           sequence that ended the previous chunk (batch, nchunks) uint8
//   status  one int32 in the last 256 bytes    0 after a clean run; a kernel that gave up a bounded wait
//                                              leaves its code here (the output is then invalid)
struct SsdScratch {
    size_t off_dt, off_dA, off_states, off_cb, off_prev16, off_aux, off_aux_state, off_aux_decay, off_seq_start, off_seq_carry, off_status, total;
    int nchunks;
};

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

inline SsdScratch ssd_scratch_layout(const mb200_ssd_args &a)
{
    SsdScratch s;
    s.nchunks = (a.seqlen + a.chunk_size - 1) / a.chunk_size;
    const size_t per = (size_t)a.batch * a.nheads * s.nchunks * a.chunk_size * sizeof(float);
    s.off_dt = 0;
    s.off_dA = align256(s.off_dt + per);
    s.off_states = align256(s.off_dA + per);
    s.off_cb = align256(s.off_states + (size_t)a.batch * s.nchunks * a.nheads * a.headdim * a.dstate * sizeof(float));
    s.off_prev16 = align256(s.off_cb + (size_t)a.batch * s.nchunks * a.ngroups * a.chunk_size * a.chunk_size * sizeof(float));
    s.off_aux = align256(s.off_prev16 + (size_t)a.batch * s.nchunks * a.nheads * a.headdim * a.dstate * 2);
    s.off_aux_state = align256(s.off_aux + (size_t)a.batch * a.nheads * s.nchunks * sizeof(float));
    s.off_aux_decay = align256(s.off_aux_state + (size_t)a.batch * a.nheads * a.headdim * a.dstate * sizeof(float));
    s.off_seq_start = align256(s.off_aux_decay + (size_t)a.batch * a.nheads * sizeof(float));
    s.off_seq_carry = align256(s.off_seq_start + (size_t)a.batch * s.nchunks * a.chunk_size);      // sizes do not depend on pointers
    s.off_status = align256(s.off_seq_carry + (size_t)a.batch * s.nchunks);
    s.total = s.off_status + 256;
    return s;
}

// Tensor-core stages (ssd_tc.cu): whether the call qualifies, and the two launch groups.  The LOCAL stages read
// x, B and dt only; the OUTPUT stages add C, z and out.  Each predicate looks at nothing else, so the two halves
// of a sequence split agree on how the LOCAL half ran although they are handed different C / z / out.
bool ssd_tc_local_eligible(const mb200_ssd_args &a);
bool ssd_tc_output_eligible(const mb200_ssd_args &a);
bool ssd_tc_cb_eligible(const mb200_ssd_args &a);      // C as the tensor-core C.B^T kernel needs it
int ssd_tc_chunk_state(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream);
// parts: 1 = the C.B^T launch, 2 = the chunk-scan launch, 3 = both
int ssd_tc_cb_and_scan(const mb200_ssd_args &a, const SsdScratch &lay, bool states_np, cudaStream_t stream, int parts = 3);
// Chunk states and inter-chunk recurrence fused (one CTA per batch row and head); leaves the 16-bit entering
// states in [n][p] order, which ssd_tc_cb_and_scan is told through states_np.
bool ssd_tc_stream_eligible(const mb200_ssd_args &a);
int ssd_tc_state_stream(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream);
// OUTPUT phase of a sequence split on that path: adds the incoming state's share to the entering states the LOCAL
// phase left (H_c += prefix_decay_c * S_in) and forms the range's end state.
int ssd_tc_apply_incoming(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream);

}  // namespace mb200
