// Types shared by the decode-attention translation units.
#pragma once

#include "tq_common.cuh"
#include "tq_step_blocks.cuh"

struct CombineArgs {
    const float *part_m, *part_l, *part_acc;
    int n_splits, Hq, G;
    // When seg_chunk > 0 the partials of KV row r are those of the CTAs whose chunk of the
    // flattened (row * seg_npad + token) space overlaps the row; otherwise all n_splits are valid.
    int seg_chunk, seg_npad;
    // When len_ptr is set the sequence length is *len_ptr + len_add (clamped to capacity) and the
    // kernel derives seg_chunk / seg_npad itself, with the plan the decode kernel used.
    const int *len_ptr;
    int len_add, capacity, plan_rows, plan_ctas, plan_step;
    // Peer gather (KV-head sharding): when gather_world > 0 the finished rows go to every rank's
    // gathered buffer instead of `out`, and every block adds its row count to this rank's word in every peer.
    int gather_world, gather_rank, gather_heads_total;
    unsigned gather_seq;
    const unsigned *gather_seq_ptr;  // when set, the step number is *gather_seq_ptr + 1 (the wait kernel stores it back)
    long long gather_out_stride;     // bytes between a rank's two gathered buffers (step s uses buffer s & 1)
    void *gather_out[TQ_MAX_PEERS];
    unsigned *gather_flags[TQ_MAX_PEERS];
    // Sequence split (fewer KV heads than ranks): `parts` ranks share a group of KV heads, each
    // holding a disjoint part of the tokens.  When parts > 0 (grouped combine, gather_world > 0) the
    // block does not finish its rows: it stores the merged partial (max, sum, acc[128], fp32,
    // rotated space) of every head into slot `part` of the partial-exchange buffer of every rank.
    int parts, part, head_group;
    int64_t exch_rows;  // rows of the whole model (batch x q_heads_total): the exchange buffer's extent
    const float *rot_v;  // R_v[d][e]
    const void *q;       // original-dtype query, for the dense tail
    void *out;
    float *out_f32;      // when set (grouped combine only), the result goes here as fp32 and `out` is not written
    int n_tail;
    const void *tail_k, *tail_v;
    int64_t tk_sb, tk_sh, tk_st, tv_sb, tv_sh, tv_st;
};

// Carved view of the caller's scratch buffer (see tq_decode_workspace_bytes).
struct DecodeWorkspace {
    float *qrot;      // [rows][128]  q @ R_k^T
    float *qproj;     // [rows][128]  q @ S^T
    float *part_m;    // [rows][splits]
    float *part_l;    // [rows][splits]
    float *part_acc;  // [rows][splits][128]
};

DecodeWorkspace tq_carve_workspace(void *workspace, int64_t rows, int n_splits);
// rows_per_step: how many rows every rank reports per step (0: batch * q_heads_total / world)
int32_t tq_launch_gather_wait(const tq_gather_desc *g, int *error_flag, int limit_ms, int32_t batch, size_t elem_bytes,
                              void *out_final, cudaStream_t stream, int64_t rows_per_step = 0);
int32_t tq_launch_qprep(tq_ctx *ctx, const void *q, int32_t q_dtype, int64_t rows, float *qrot, float *qproj,
                        cudaStream_t stream);
// Query preparation for the tensor-core kernel; with `append` the same launch also encodes and
// appends the step's new key / value vectors.
int32_t tq_launch_qprep_frag(tq_ctx *ctx, const void *q, int32_t q_dtype, int64_t kv_rows, int G, uint32_t *frag,
                             const TqPackArgs *append, cudaStream_t stream);
// `programmatic`: launch as a programmatic dependent of the preceding kernel (honoured by the
// grouped variant, which waits for that kernel before it reads the partials).
int32_t tq_launch_combine(const CombineArgs &a, int32_t q_dtype, int64_t rows, cudaStream_t stream,
                          bool programmatic = false);
