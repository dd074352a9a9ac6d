// Types shared by the decode-attention translation units.
#pragma once

#include "tq_common.cuh"

struct CombineArgs {
    const float *part_m, *part_l, *part_acc;
    int n_splits, Hq, G;
    // When seg_chunk > 0 the partials of KV row r are those of the CTAs whose chunk of the
    // flattened (row * seg_npad + token) space overlaps the row; otherwise all n_splits are valid.
    int seg_chunk, seg_npad;
    const float *rot_v;  // R_v[d][e]
    const void *q;       // original-dtype query, for the dense tail
    void *out;
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

// Words per query head in the fragment area written by tq_qprep_frag_kernel (8 lane variants of
// 26 words, padded to the size of the rotated + projected query rows it overlays).
#define TQ_FRAG_ROW_WORDS (2 * TQ_D + 8)

DecodeWorkspace tq_carve_workspace(void *workspace, int64_t rows, int n_splits);
int32_t tq_launch_qprep(tq_ctx *ctx, const void *q, int32_t q_dtype, int64_t rows, float *qrot, float *qproj,
                        cudaStream_t stream);
int32_t tq_launch_qprep_frag(tq_ctx *ctx, const void *q, int32_t q_dtype, int64_t kv_rows, int G, uint32_t *frag,
                             cudaStream_t stream);
int32_t tq_launch_combine(const CombineArgs &a, int32_t q_dtype, int64_t rows, cudaStream_t stream);
