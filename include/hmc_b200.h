/*
 * hmc_b200.h -- C ABI of libhmc_b200.so: the B200 (sm_100a) kernels behind the hyper_multicore
 * MegaMoE / MegaGate / MegaMHC operator boundary.
 *
 * Conventions (all entry points):
 *   - plain device pointers, 64-bit extents, a `void* stream` that is a cudaStream_t (NULL = legacy
 *     default stream); work is enqueued on that stream and the call returns before completion;
 *   - the caller owns and pre-allocates every buffer, as at the reference's operator boundary
 *     (hyper_multicore/torch/ops.py wrappers allocate, torch/csrc impls only check and launch);
 *   - the return value is 0 or a negative HMC_ERR_* code; hmc_last_error() then describes the
 *     failed check for the calling thread. Nothing throws and nothing synchronises the device;
 *   - device-side failures (a bounded wait that ran out) are written to the caller's int32
 *     `status` words; word 0 is 0 while healthy (HMC_STATUS_*).
 *
 * Reference citations name files of mindspore-ai/hyper-multicore by their path in that project.
 */
#ifndef HMC_B200_H_
#define HMC_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HMC_ABI_VERSION 1

/* host-side return codes */
#define HMC_OK 0
#define HMC_ERR_INVALID (-1) /* argument check failed (maps to ValueError / RuntimeError) */
#define HMC_ERR_CUDA (-2)    /* a CUDA runtime or driver call failed */
#define HMC_ERR_LIMIT (-3)   /* a documented size limit was exceeded */

/* device status words */
#define HMC_STATUS_WORDS 8
#define HMC_STATUS_OK 0
#define HMC_STATUS_TIMEOUT_PIPELINE 1 /* an intra-kernel barrier wait ran out: {role, stage, k} */
#define HMC_STATUS_TIMEOUT_ARRIVAL 2  /* rows of a group never arrived: {group, expected, seen} */
#define HMC_STATUS_TIMEOUT_READY 3    /* a peer never published "ready": {peer, expected, seen} */
#define HMC_STATUS_BAD_INDEX 4        /* an expert id or mapping entry was out of range */

const char* hmc_last_error(void);
int hmc_abi_version(void);
/* Transport / queue layout versions the reference's loader asserts
 * (hyper_multicore/torch/csrc/registration.cpp:21-22). */
int hmc_mega_moe_transport_version(void);
int hmc_worker_queue_layout_version(void);
/* Measurement helpers, no counterpart in the reference. hmc_launch_count: kernels this library has launched
 * in this process. While hmc_profile_enable(1) is in force, every call of the entry points listed below is
 * bracketed by two CUDA events on its stream; hmc_profile_collect waits for them, adds the device time and the
 * number of calls per kind into ms_by_kind / calls_by_kind [kinds] and forgets them (it synchronises).
 * hmc_profile_enable_kinds(mask) brackets only the kinds whose bit (1 << HMC_PROFILE_*) is set, so that a timed
 * region can carry the events of its dominant kernel alone. */
#define HMC_PROFILE_GROUPED_GEMM 0 /* hmc_grouped_gemm */
#define HMC_PROFILE_MX_GEMM 1      /* hmc_mx_gemm */
#define HMC_PROFILE_MX_QUANT 2     /* hmc_mx_quant */
#define HMC_PROFILE_EP 3           /* hmc_ep_dispatch, hmc_ep_pull, hmc_ep_combine, hmc_ep_wait(_groups), count exchange */
#define HMC_PROFILE_ROUTE 4        /* route preparation and token (un)permutation entry points */
#define HMC_PROFILE_KINDS 5
int64_t hmc_launch_count(void);
int hmc_profile_enable(int on);
int hmc_profile_enable_kinds(uint32_t kinds_mask);
int hmc_profile_collect(double* ms_by_kind, int64_t* calls_by_kind, int kinds);
/* Like hmc_profile_collect, but returns the calls one by one in the order they were made: kind, start (ms after
 * the first call's start) and duration of up to `capacity` calls. Returns the number of calls written. */
int hmc_profile_dump(int32_t* kinds, double* start_ms, double* duration_ms, int capacity);

/* ------------------------------------------------------------------------------------------
 * Grouped expert GEMM (tcgen05 + TMA + TMEM).
 * Replaces: GMM1/GMM2 Cube tasks ExecuteGroupedMatmul
 * (hyper_multicore/ops/hyper_mega_moe/op_kernel/worker_kernel.cpp:225-299), the arch35 BF16
 * worker (hyper_multicore/ops/common/mega_moe/adapters/arch35/gmm/bf16_worker.h:44-85), the
 * SwiGLU task (worker_kernel.cpp:122-223) and SwiGLUGrad
 * (hyper_multicore/ops/hyper_mega_moe_grad/op_kernel/worker_kernel.cpp:164-195).
 * ------------------------------------------------------------------------------------------ */
#define HMC_GEMM_RAGGED_M 0 /* C[rows_g, n] = A[rows_g, k] * B_g ; rows_g from group_ends */
#define HMC_GEMM_RAGGED_K 1 /* C_g[m, n] = A[rows_g, m]^T * B[rows_g, n] (weight gradients) */
#define HMC_MAJOR_K 0       /* operand stored with the contraction index contiguous */
#define HMC_MAJOR_MN 1      /* operand stored with the M/N index contiguous */
#define HMC_TILE_AUTO 0
#define HMC_TILE_SINGLE 1
#define HMC_TILE_PAIR 2
#define HMC_EPI_STORE_BF16 0
#define HMC_EPI_STORE_F32 1   /* FP32 output (partial weight gradients, mHC projection) */
#define HMC_EPI_SWIGLU 2      /* B has 2n columns [gate | up]; c = U[rows, 2n], aux = Act[rows, n] */
#define HMC_EPI_SWIGLU_GRAD 3 /* acc = dAct[rows, n]; aux = U[rows, 2n] (input); c = dU[rows, 2n] */
#define HMC_EPI_SWIGLU_GRAD_MXQ 5 /* hmc_mx_gemm only: acc = dAct[rows, n]; aux = U[rows, 2n]; dU = [dgate | dup] leaves the
                                    epilogue quantised along both axes (hmc_mx_quant's HMC_MXQ_SWIGLU_GRAD); c = dAct is
                                    optional */
#define HMC_EPI_SWIGLU_MXQ 4  /* hmc_mx_gemm only: c = U[rows, n] with n = 2 * width, and bf16(silu(gate) * up) leaves the
                                 epilogue quantised along both axes (what hmc_mx_quant's HMC_MXQ_SWIGLU would make of U) */
#define HMC_CLAMP_NONE 0
#define HMC_CLAMP_BEFORE_SILU 1 /* silu(min(g, L)) * clamp(u, -L, L) */
#define HMC_CLAMP_AFTER_SILU 2  /* min(silu(g), L) * clamp(u, -L, L) */

/* Optional: the result rows of a RAGGED_M / STORE_BF16 GEMM leave the epilogue straight for the routed
 * buffers of their source ranks (the reference's combine stage, tasks/alltoall.py:90-157 and
 * worker_kernel.cpp:301-366, fused into the GEMM that produces the rows). Row r of local expert g came
 * from source s = last s with segment_start[g * ep + s] <= r and goes to row
 * combine_target_off[s * local_experts + g] + (r - segment_start[g * ep + s]) of peer_buffers[s].
 * Every (32-row, half-tile) piece adds its row count to the destination's HMC_CTRL_COMBINE counter with
 * release semantics, so a source has all its rows once the counter reaches
 * rows * hmc_grouped_gemm_combine_units(n). */
typedef struct hmc_gemm_combine {
  const int64_t* segment_start;      /* device [local_experts * ep], from hmc_route_offsets */
  const int64_t* combine_target_off; /* device [ep * local_experts] */
  void* const* peer_buffers;         /* host array [ep]: routed buffer of every rank, as mapped here */
  void* const* peer_ctrl;            /* host array [ep]: control block of every rank */
  int64_t ep;
  int64_t local_experts;             /* must equal the GEMM's groups */
  int64_t target_rows_limit;
} hmc_gemm_combine;

struct hmc_ep_dispatch_args; /* defined with the expert-parallel transport below */

typedef struct hmc_grouped_gemm_args {
  int32_t mode;
  int32_t a_major; /* RAGGED_M: HMC_MAJOR_K. RAGGED_K: HMC_MAJOR_MN */
  int32_t b_major; /* RAGGED_M: MN = B[groups, k, n_cols], K = B[groups, n_cols, k] */
  int32_t epilogue;
  int32_t groups;
  int32_t max_ctas; /* 0 = one CTA per SM */
  int32_t tile_mode; /* HMC_TILE_AUTO, _SINGLE (128-row tiles) or _PAIR (256-row CTA-pair tiles; RAGGED_K: where m % 256 == 0) */
  int32_t swiglu_clamp; /* HMC_CLAMP_*: SwiGLU / SwiGLU-grad epilogues only */
  int64_t rows;     /* extent of the ragged dimension of a (and of b for RAGGED_K) */
  int64_t m;        /* RAGGED_K only */
  int64_t n;
  int64_t k; /* RAGGED_M only */
  const void* a;
  const void* b;
  void* c;
  void* aux;
  const int64_t* group_ends;  /* device int64[groups], cumulative row ends (reference group_list) */
  const int32_t* ready_counters; /* optional device int32[groups]: rows landed per group */
  uint64_t ready_budget_ns;      /* 0 = 10 s */
  int32_t* status;               /* optional device int32[HMC_STATUS_WORDS] */
  /* Numerics options of the reference (hyper_multicore/modules/mega_moe/numerics.py:21-50,
   * docs/mega_moe.md:258-308; device math ops/common/mega_moe/routing_probabilities.h:19-108). */
  float swiglu_limit;     /* L of the clamp: gate clipped from above, up clipped to [-L, L] */
  int32_t reserved;
  const float* row_probs; /* optional device float[rows]: routing probability of each row ("before FC2").
                             SWIGLU: aux = bf16(fp32(bf16(act)) * p). SWIGLU_GRAD: the accumulator is the
                             gradient of that weighted activation; dAct = bf16(fp32(bf16(acc)) * p) */
  float* row_dot;         /* SWIGLU_GRAD with row_probs: row_dot[row] += sum_col bf16(act) * bf16(acc), the
                             probability gradient; zeroed by the caller */
  const hmc_gemm_combine* combine; /* optional, RAGGED_M + STORE_BF16: c is ignored, rows go to their sources */
  uint64_t pipe_budget_ns;         /* bound of the kernel's internal barrier waits, 0 = 4 s. With ready_counters the
                                      consumer-side waits add ready_budget_ns to it: while the producer is allowed to
                                      wait for late rows, the warps behind it must not give up first */
  /* Optional, RAGGED_M with ready_counters: this launch also SENDS this rank's rows. Extra warps of every CTA
   * execute the push dispatch described here (peer stores + arrival counters, exactly what hmc_ep_dispatch
   * does) while the tile producer waits per expert for the rows this rank receives, so the NVLink transfer
   * overlaps the first tiles instead of preceding them: the reference runs its dispatch PUT tasks and GMM1
   * inside one launch the same way (ops/hyper_mega_moe/op_kernel/worker_kernel.cpp:301-366,
   * tasks/gmm.py:154-160). `a` must be this rank's own receive buffer, ready_counters its arrival counters,
   * dispatch->local_experts == groups and dispatch->hidden == k. Every CTA of the launch is resident at once
   * (one per SM), so a CTA waiting for rows never keeps another CTA's dispatch warps from running. */
  const struct hmc_ep_dispatch_args* dispatch;
  const int32_t* skip_flag;        /* optional device int32: when it holds a non-zero value as the kernel starts, the
                                      launch does nothing (no tiles, no dispatch). Set by hmc_route_guard when the
                                      call it belongs to must not run (see there) */
} hmc_grouped_gemm_args;

int hmc_grouped_gemm(const hmc_grouped_gemm_args* args, void* stream);
/* Counter increments per result row of a fused-combine GEMM with n output columns. */
int64_t hmc_grouped_gemm_combine_units(int64_t n);

/* ------------------------------------------------------------------------------------------
 * MXFP8 expert GEMM (tcgen05 kind::mxf8f6f4.block_scale) and its quantisers.
 * Replaces the reference's MX GMM worker ExecuteMxGmmMatrix
 * (hyper_multicore/ops/common/mega_moe/adapters/arch35/gmm/mxfp8_worker.h:15-159, descriptor
 * contracts/mx_gmm_descriptor.h:18-87) and the dual-axis MX quantiser ExecuteMxQuantRange
 * (adapters/arch35/quantization/dual_axis_mxfp8_worker.h:23-110, kinds plain / SwiGLU+quant /
 * SwiGLUGrad+quant; graph hyper_multicore/modules/mega_moe/backends/mxfp8/graph.py:116-180).
 *
 * Operands are E4M3 with one UE8M0 scale per 32 elements along the contraction axis.
 * Activations use a PADDED expert-major layout: the rows of group g start at 128 * (number of
 * 128-row blocks of the groups before it), padding rows are zero, so that 128-row tiles, 32-row
 * scale blocks and scale-factor atoms never straddle two experts.
 * Scale factors are stored as 512-byte atoms covering 128 rows (or columns) x 4 consecutive
 * 32-element blocks: byte (r % 32) * 16 + (r / 32) * 4 + kk, the layout tcgen05.cp expects.
 *   row-quantised activations : atoms [k / 128][pad_blocks]        (contraction along the row)
 *   col-quantised activations : atoms [pad_blocks][width / 128]     (contraction along the rows)
 *   weights, forward          : atoms [groups][k / 128][n / 128]
 * pad_blocks is the caller's upper bound ceil(rows / 128) + groups; buffers are sized with it.
 * Limits: k, n (and m for RAGGED_K) multiples of 128.
 * ------------------------------------------------------------------------------------------ */
typedef struct hmc_mx_gemm_args {
  int32_t mode;     /* HMC_GEMM_RAGGED_M or HMC_GEMM_RAGGED_K */
  int32_t b_major;  /* RAGGED_M: MN = b[groups, k, n], K = b[groups, n, k]. RAGGED_K: ignored */
  int32_t epilogue; /* HMC_EPI_STORE_BF16, HMC_EPI_STORE_F32 (RAGGED_K only), HMC_EPI_SWIGLU_MXQ or
                       HMC_EPI_SWIGLU_GRAD_MXQ (RAGGED_M only) */
  int32_t groups;
  int32_t max_ctas;
  int32_t tile_mode;  /* HMC_TILE_AUTO, _SINGLE (128 x 128 tiles) or _PAIR (256 x 256 CTA-pair tiles; needs n % 256 == 0,
                         and m % 256 == 0 for RAGGED_K). AUTO takes pairs wherever the shape allows them. */
  int64_t rows;       /* un-padded rows (sum of the groups) */
  int64_t pad_blocks; /* 128-row blocks the padded activation buffers hold */
  int64_t m;          /* RAGGED_K only */
  int64_t n;
  int64_t k;          /* RAGGED_M only */
  const void* a;      /* RAGGED_M: e4m3 [pad_blocks*128, k] row-quantised. RAGGED_K: e4m3 [pad_blocks*128, m] col-quantised */
  const void* a_scale;
  const void* b;      /* RAGGED_M: weight data. RAGGED_K: e4m3 [pad_blocks*128, n] col-quantised */
  const void* b_scale;
  void* c;            /* RAGGED_M: bf16 [rows, n] in the UN-padded layout. RAGGED_K: [groups, m, n] */
  const int64_t* group_ends; /* device int64[groups], cumulative un-padded row ends */
  int32_t* status;
  const hmc_gemm_combine* combine; /* optional, RAGGED_M: rows go to their source ranks (see hmc_gemm_combine);
                                      c may then be NULL; counter units per row: hmc_mx_gemm_combine_units(n) */
  /* HMC_EPI_SWIGLU_MXQ (RAGGED_M, b_major MN, CTA-pair tiles): the quantised activation in the layouts of
   * hmc_mx_quant_args, width = n / 2: e4m3 [pad_blocks*128, width] twice and their scale atoms (the column pair may
   * be NULL). */
  void* act_row_data;
  void* act_row_scale;
  void* act_col_data;
  void* act_col_scale;
  /* HMC_EPI_SWIGLU_GRAD_MXQ (RAGGED_M, b_major K, CTA-pair tiles): aux = the saved U [rows, 2n] bf16; the four
   * outputs above receive dU, width = 2n; c (dAct, bf16 [rows, n]) may be NULL. */
  const void* aux;
  const int32_t* skip_flag; /* optional device word: non-zero when the launch runs = the launch does nothing (see
                               hmc_route_guard) */
} hmc_mx_gemm_args;

int hmc_mx_gemm(const hmc_mx_gemm_args* args, void* stream);
int64_t hmc_mx_gemm_combine_units(int64_t n);

#define HMC_MXQ_PLAIN 0       /* quantise src[rows, width] */
#define HMC_MXQ_SWIGLU 1      /* src = U[rows, 2*width]; quantise bf16(silu(gate) * up) */
#define HMC_MXQ_SWIGLU_GRAD 2 /* src = dAct[rows, width/2], aux = U[rows, width]; quantise dU = [dgate | dup] */

typedef struct hmc_mx_quant_args {
  int32_t kind;   /* HMC_MXQ_* */
  int32_t groups;
  int64_t rows;
  int64_t pad_blocks;
  int64_t width;  /* columns of the quantised result (multiple of 128) */
  const void* src;            /* bf16, un-padded expert-major rows */
  const void* aux;            /* bf16 U for HMC_MXQ_SWIGLU_GRAD */
  const int64_t* group_ends;
  void* row_data;             /* optional out: e4m3 [pad_blocks*128, width], 32-blocks along the row */
  void* row_scale;            /* atoms [width/128][pad_blocks] */
  void* col_data;             /* optional out: e4m3 [pad_blocks*128, width], 32-blocks down the rows */
  void* col_scale;            /* atoms [pad_blocks][width/128] */
  void* dense;                /* optional out: bf16 [rows, width] un-padded (the un-quantised result) */
  const int32_t* skip_flag;   /* optional device word: non-zero when the launch runs = the launch does nothing */
} hmc_mx_quant_args;

int hmc_mx_quant(const hmc_mx_quant_args* args, void* stream);

/* Weight helpers. hmc_mx_quant_weight produces the reference's physical fields
 * (docs/mega_moe.md:169-200): col_data/col_scale [e, m/64, n, 2] (blocks along m) and
 * row_data/row_scale [e, m, n/64, 2] (blocks along n) from a bf16 weight [e, m, n].
 * hmc_mx_pack_weight_scale converts one of those scale tensors into the GEMM's atoms:
 * axis 0 (col_scale): atoms [e][m/128][n/128] with the atom row = n; axis 1 (row_scale):
 * atoms [e][n/128][m/128] with the atom row = m. */
int hmc_mx_quant_weight(const void* weight_bf16, int64_t experts, int64_t m, int64_t n, void* col_data,
                        void* col_scale, void* row_data, void* row_scale, void* stream);
int hmc_mx_pack_weight_scale(const void* scale, int axis, int64_t experts, int64_t m, int64_t n, void* atoms,
                             void* stream);

/* ------------------------------------------------------------------------------------------
 * MegaGate.
 * hmc_gate_route replaces torch.ops.hyper_multicore.mega_gate_route(_out)
 * (hyper_multicore/torch/csrc/mega_gate_registration.cpp:10-27, checks mega_gate.cpp:40-61, device
 * pipeline hyper_multicore/ops/hyper_mega_gate/op_kernel/route_pipeline.h:73-562) and extends it
 * to the softmax and sigmoid scoring of MegaGate._torch_forward
 * (hyper_multicore/modules/mega_gate/module.py:189-227).
 * hmc_gate_route_grad replaces mega_gate_route_grad (mega_gate_registration.cpp:29-41,
 * mega_gate.cpp:132-176, route_grad_pipeline.h:138-191, hyper_mega_gate_route_grad_post.cpp:59-140).
 * hmc_gate_project is the FP32 router projection F.linear(x.float(), W.float())
 * (hyper_multicore/modules/mega_gate/function.py:175-178).
 * ------------------------------------------------------------------------------------------ */
#define HMC_SCORE_SQRTSOFTPLUS 0
#define HMC_SCORE_SOFTMAX 1
#define HMC_SCORE_SIGMOID 2

typedef struct hmc_gate_route_args {
  const float* logits;       /* [tokens, experts] */
  const float* text_bias;    /* [experts] selection-only correction bias */
  const float* vision_bias;  /* [experts], used where image_mask is true */
  const uint8_t* image_mask; /* [tokens] bool, or NULL when use_vision_bias == 0 */
  int32_t use_vision_bias;
  int32_t experts;
  int32_t top_k;
  int32_t scoring; /* HMC_SCORE_* */
  int64_t tokens;
  float scale; /* routed_scaling_factor */
  float* weights;      /* out [tokens, top_k] */
  int64_t* indices;    /* out [tokens, top_k], descending biased score, ties to the lower id */
  float* route_scores; /* out [tokens, experts] unbiased scores (saved for backward) */
  float* selected;     /* out [tokens, top_k] unbiased scores of the winners */
  float* denominator;  /* out [tokens, 1] sum(selected) + 1e-20 */
  /* Group-limited selection. NOT part of the reference (it has no expert groups); an extension for
   * routers that restrict each token to a few expert groups. experts are split into n_group equal,
   * contiguous groups; a group's score is the sum of its two largest biased scores (its largest one
   * for groups of one expert); only experts of the topk_group best groups (ties to the lower group)
   * take part in the top-k. n_group == 0 switches the limit off. n_group <= 32. */
  int32_t n_group;
  int32_t topk_group;
} hmc_gate_route_args;

typedef struct hmc_gate_route_grad_args {
  const float* logits;
  const float* route_scores;
  const float* selected;
  const float* denominator;
  const int64_t* indices;
  const float* grad_weights; /* [tokens, top_k] */
  int32_t experts;
  int32_t top_k;
  int32_t scoring;
  int32_t reserved;
  int64_t tokens;
  float scale;
  float* grad_logits; /* out [tokens, experts] */
  int32_t* status;    /* optional */
} hmc_gate_route_grad_args;

int hmc_gate_route(const hmc_gate_route_args* args, void* stream);
int hmc_gate_route_grad(const hmc_gate_route_grad_args* args, void* stream);
int hmc_gate_project(const void* x, int x_is_bf16, const void* w, int w_is_bf16, int64_t tokens, int64_t hidden,
                     int64_t experts, float* logits, void* stream);
/* Same projection on tcgen05 for BF16 hidden states: the weight is split into three BF16 parts that
 * sum to its FP32 value, so the result keeps FP32 accuracy. Scratch comes from the caller. */
int64_t hmc_gate_project_workspace_bytes(int64_t tokens, int64_t hidden, int64_t experts);
int hmc_gate_project_tc(const void* x_bf16, const void* w, int w_is_bf16, int64_t tokens, int64_t hidden,
                        int64_t experts, float* logits, void* workspace, int64_t workspace_bytes, void* stream);

/* tcgen05 projection with a bounded accumulation chain: the dominant BF16 part of the weight accumulates in
 * the tensor core for 128 elements of K at a time and is promoted into FP32 registers in between, which
 * keeps the result within the reference's logits tolerance (1e-5 / 1e-6). One kernel after the weight
 * split; workspace = three BF16 parts of the weight, padded to 64 experts. A caller that keeps the workspace
 * between calls may pass w = NULL while the weight is unchanged: the split is then skipped and the parts of the
 * earlier call are used (w_is_bf16 must be the same as in that call). status (optional, HMC_STATUS_WORDS)
 * receives pipeline time-outs. */
int64_t hmc_gate_project_promoted_workspace_bytes(int64_t hidden, int64_t experts);
int hmc_gate_project_promoted(const void* x_bf16, const void* w, int w_is_bf16, int64_t tokens, int64_t hidden,
                              int64_t experts, float* logits, void* workspace, int64_t workspace_bytes,
                              int32_t* status, void* stream);

/* The same projection followed, in the same launch, by the Route of every token (MegaGate.forward,
 * hyper_multicore/modules/mega_gate/module.py:189-227, as one device pass): with at most 64 experts and no group
 * limit (hmc_gate_project_route_supported) a thread of the projection's epilogue holds a token's whole logits row and
 * scores, biases, selects and weighs it there. route->logits is ignored - the logits computed here are routed and
 * also written to `logits`; route->tokens and route->experts give the extents; every output of hmc_gate_route is
 * produced, bit for bit what hmc_gate_project_promoted followed by hmc_gate_route writes. workspace, w == NULL and
 * status as for hmc_gate_project_promoted. */
int hmc_gate_project_route_supported(int64_t experts, int32_t n_group);
int hmc_gate_project_route(const void* x_bf16, const void* w, int w_is_bf16, int64_t hidden, float* logits,
                           void* workspace, int64_t workspace_bytes, const hmc_gate_route_args* route, int32_t* status,
                           void* stream);

/* ------------------------------------------------------------------------------------------
 * MoE route preparation and token (un)permutation.
 * hmc_moe_histogram         : _resolve_counts (hyper_multicore/modules/mega_moe/route.py:186-211)
 * hmc_moe_sort_routes       : the expert-major permutation index of npu_moe_init_routing_v2 /
 *                             npu_moe_token_permute (route.py:266-295) as a stable counting sort over
 *                             the flat index token * top_k + slot; mapping[flat] = destination row
 * hmc_moe_gather_rows       : payload half of moe_token_permute_out
 *                             (hyper_multicore/torch/csrc/moe_token_permute_out.cpp:50-60)
 * hmc_moe_permute_from_mapping : moe_token_permute_from_mapping_out
 *                             (hyper_multicore/ops/common/mega_moe/utilities.asc:162-209)
 * hmc_moe_unpermute         : restore_topk_output (route.py:1029-1051), rounding as in the golden
 *                             (tests/common/multicore/moe_reference.py:179-180)
 * hmc_moe_unpermute_grad    : mega_moe_unpermute_grad_out (torch/csrc/mega_moe_unpermute.cpp:56-65)
 * hmc_moe_token_permute_grad: moe_token_permute_grad (torch/csrc/moe_token_permute_grad.cpp:29-38); a token's
 *                             rows are added in descending row (= expert) order with a BF16 rounding per
 *                             addition, the order torch.autograd gives the golden
 *                             (tests/common/multicore/moe_reference.py:170-181)
 * hmc_zero_empty_expert_grad: zero_empty_expert_grad_ (torch/csrc/mega_moe_utilities.cpp:64-92)
 * hmc_route_offsets         : route_offsets / _compute_route_metadata, push mode
 *                             (route.py:309-390, utilities.asc:89-151); row units. totals =
 *                             {rows routed by this rank, rows received by this rank};
 *                             recv_segment_start[le * ep + s] = first received row of (le, s);
 *                             send_order_start[experts + 1] (optional) = prefix of this rank's segments in the
 *                             order a GEMM-carried dispatch sends them: local expert 0 of every destination
 *                             (rank + 1 first, this rank last), then local expert 1, ...
 *                             (the reference rotates destinations the same way, scheduler/scheduler.py:27-53)
 * ------------------------------------------------------------------------------------------ */
int64_t hmc_moe_sort_workspace_bytes(int64_t entries, int64_t experts);
int hmc_moe_histogram(const void* indices, int indices_are_i64, int64_t entries, int64_t experts, int32_t* counts,
                      int32_t* status, void* stream);
int hmc_moe_sort_routes(const void* indices, int indices_are_i64, int64_t entries, int64_t experts, void* workspace,
                        int64_t workspace_bytes, int32_t* mapping, int32_t* source_of_row, int32_t* expert_of_row,
                        int32_t* counts, int64_t* cumulative, int32_t* status, void* stream);
/* No counterpart in the reference: an allocation-free variant of hmc_moe_sort_routes for callers that
 * cannot obtain device memory when they route (a frozen memory pool, a plugin that was handed a fixed
 * set of buffers, a latency-critical loop where cudaMalloc may stall the device). Its scratch is a
 * built-in device array of HMC_SORT_STATIC_BYTES that every GPU loading the library keeps until exit.
 *  - limit: hmc_moe_sort_workspace_bytes(entries, experts) <= HMC_SORT_STATIC_BYTES, i.e.
 *    ceil(entries / 1024) * experts <= 1 Mi (for example 1 Mi routes over 1024 experts); larger
 *    problems return HMC_ERR_LIMIT and must use hmc_moe_sort_routes;
 *  - the first call on each device looks up the array's device address (with that device current);
 *    make that first call before any stream capture begins. The address is remembered per CURRENT
 *    device: `stream` must belong to the current device. The first calls of two host threads may both
 *    do the look-up (they store the same value). The remembered address does not survive
 *    cudaDeviceReset: do not call this entry point on a device after resetting it;
 *  - all calls on a device share the array: two calls whose kernels overlap on the GPU (different
 *    streams, no ordering) race on it. Calls ordered on one stream are safe, and nothing needs
 *    clearing between them;
 *  - calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs are the
 *    caller's, with the same meaning as in hmc_moe_sort_routes. */
#define HMC_SORT_STATIC_BYTES (4 * 1024 * 1024)
int hmc_moe_sort_routes_static(const void* indices, int indices_are_i64, int64_t entries, int64_t experts,
                               int32_t* mapping, int32_t* source_of_row, int32_t* expert_of_row, int32_t* counts,
                               int64_t* cumulative, int32_t* status, void* stream);
int hmc_moe_gather_rows(const void* tokens, const int32_t* source_of_row, int64_t rows, int64_t top_k,
                        int64_t hidden, void* out, void* stream);
int hmc_moe_permute_from_mapping(const void* tokens, const int32_t* mapping, const float* probs, int64_t num_tokens,
                                 int64_t top_k, int64_t hidden, void* out, float* out_probs, int32_t* status,
                                 void* stream);
int hmc_moe_unpermute(const void* permuted, const int32_t* mapping, const float* probs, int64_t num_tokens,
                      int64_t top_k, int64_t hidden, int64_t permuted_rows, void* out, int32_t* status, void* stream);
int hmc_moe_unpermute_grad(const void* permuted, const void* grad_out, const int32_t* mapping, const float* probs,
                           int64_t num_tokens, int64_t top_k, int64_t hidden, void* grad_permuted, float* grad_probs,
                           int32_t* status, void* stream);
int hmc_moe_token_permute_grad(const void* grad_permuted, const int32_t* mapping, int64_t num_tokens, int64_t top_k,
                               int64_t hidden, void* grad_tokens, int32_t* status, void* stream);
int hmc_zero_empty_expert_grad(void* first, int64_t first_bytes_per_expert, void* second,
                               int64_t second_bytes_per_expert, const int64_t* cumulative, int64_t experts,
                               void* stream);
int hmc_route_offsets(const int32_t* counts, int64_t ep, int64_t experts, int64_t rank, int64_t* dispatch_src_off,
                      int64_t* dispatch_target_off, int32_t* dispatch_size, int64_t* combine_src_off,
                      int64_t* combine_target_off, int32_t* combine_size, int64_t* group_list, int64_t* totals,
                      int64_t* recv_segment_start, int64_t* send_order_start, void* stream);

/* ------------------------------------------------------------------------------------------
 * MegaMHC.
 * hmc_mega_mhc replaces torch.ops.hyper_multicore.mega_mhc
 * (hyper_multicore/torch/csrc/registration_mhc.cpp:19-33, mega_mhc.cpp:40-96, device worker
 * hyper_multicore/ops/hyper_mega_mhc/op_kernel/worker_kernel.cpp:92-268); hmc_mega_mhc_grad replaces
 * mega_mhc_grad (registration_mhc.cpp:35-49, hyper_multicore/ops/hyper_mega_mhc_grad/op_kernel/
 * worker_kernel.cpp). Shapes are the flattened token-major ones: activations [tokens, (4,) hidden]
 * BF16, coefficients FP32. The caller provides scratch (see the *_workspace_bytes functions).
 * ------------------------------------------------------------------------------------------ */
typedef struct hmc_mega_mhc_args {
  int64_t tokens;
  int64_t hidden;
  const void* previous_output;        /* [tokens, hidden] bf16 */
  const void* residual;               /* [tokens, 4, hidden] bf16 */
  const float* previous_pre_mix;      /* [tokens, 4] */
  const float* previous_post_mix;     /* [tokens, 4] */
  const float* previous_residual_mix; /* [tokens, 4, 4] */
  const float* phi;                   /* [24, 4 * hidden] */
  const float* alpha;                 /* [3] */
  const float* bias;                  /* [24] */
  const void* norm_weight;            /* [hidden] bf16 */
  void* new_residual;                 /* out [tokens, 4, hidden] bf16 */
  float* next_pre_mix;                /* out [tokens, 4] */
  float* next_post_mix;               /* out [tokens, 4] */
  float* next_residual_mix;           /* out [tokens, 16] */
  void* block_input;                  /* out [tokens, hidden] bf16 */
  float* hc_before_norm;              /* cache [tokens, 24], may be NULL when need_backward == 0 */
  float* inv_rms;                     /* cache [tokens] */
  float* sum_out;                     /* cache [2 * iters, tokens, 4] or NULL */
  float* norm_out;                    /* cache [2 * iters, tokens, 16] or NULL */
  void* mixed_input;                  /* cache [tokens, hidden] bf16 (always written) */
  float* rms_rstd;                    /* cache [tokens] */
  void* workspace;
  int64_t workspace_bytes;
  float hc_eps;
  float norm_eps;
  int32_t num_iters;
  int32_t need_backward;
  int32_t* status; /* optional */
} hmc_mega_mhc_args;

typedef struct hmc_mega_mhc_grad_args {
  int64_t tokens;
  int64_t hidden;
  const void* grad_new_residual;       /* [tokens, 4, hidden] bf16 */
  const float* grad_next_pre_mix;      /* [tokens, 4] */
  const float* grad_next_post_mix;     /* [tokens, 4] */
  const float* grad_next_residual_mix; /* [tokens, 16] */
  const void* grad_block_input;        /* [tokens, hidden] bf16 */
  const void* new_residual;            /* forward output */
  const float* hc_before_norm;         /* forward caches */
  const float* inv_rms;
  const void* mixed_input;
  const float* rms_rstd;
  const void* previous_output; /* forward inputs */
  const void* residual;
  const float* previous_pre_mix;
  const float* previous_post_mix;
  const float* previous_residual_mix;
  const float* phi;
  const float* alpha;
  const float* bias;
  const void* norm_weight;
  void* grad_residual;               /* out [tokens, 4, hidden] bf16 */
  float* grad_phi;                   /* out [24, 4 * hidden] */
  float* grad_alpha;                 /* out [3] */
  float* grad_bias;                  /* out [24] */
  void* grad_previous_output;        /* out [tokens, hidden] bf16 */
  float* grad_previous_pre_mix;      /* out [tokens, 4] */
  float* grad_previous_post_mix;     /* out [tokens, 4] */
  float* grad_previous_residual_mix; /* out [tokens, 16] */
  float* grad_norm_weight;           /* out [hidden] fp32 */
  void* workspace;
  int64_t workspace_bytes;
  float hc_eps;
  int32_t num_iters;
  int32_t* status; /* optional */
} hmc_mega_mhc_grad_args;

int64_t hmc_mega_mhc_workspace_bytes(int64_t tokens, int64_t hidden);
int64_t hmc_mega_mhc_grad_workspace_bytes(int64_t tokens, int64_t hidden);
int hmc_mega_mhc(const hmc_mega_mhc_args* args, void* stream);
int hmc_mega_mhc_grad(const hmc_mega_mhc_grad_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Expert-parallel transport over CUDA-IPC peer mappings (one process per GPU, one box).
 * Replaces the reference's private SHMEM heap and its device data plane on the MoE path:
 * shmem.empty/free (hyper_multicore/shmem/_api.py:77-182), dispatch / combine PUT tasks with
 * per-expert signal ADD (hyper_multicore/ops/hyper_mega_moe/op_kernel/worker_kernel.cpp:301-366,
 * hyper_multicore/ops/common/mega_moe/transport_task.h:37-79, hyper_multicore/tasks/alltoall.py:
 * 90-157) and the ready handshake (ops/common/mega_moe/invocation_protocol.h:9-52).
 *
 * Control block (int32 words, one per rank, inside the peer-mapped allocation):
 *   [HMC_CTRL_ARRIVAL + e]              rows that have landed for local expert e (zeroed per call)
 *   [HMC_CTRL_COMBINE]                  result rows that have come back to this source (zeroed per call)
 *   [HMC_CTRL_READY + p * STRIDE]       last generation peer p declared itself ready for (never zeroed)
 * ------------------------------------------------------------------------------------------ */
#define HMC_MAX_EP 16
#define HMC_IPC_HANDLE_BYTES 64
#define HMC_CTRL_ARRIVAL 0
#define HMC_CTRL_MAX_LOCAL_EXPERTS 1024
#define HMC_CTRL_COMBINE 1024
#define HMC_CTRL_READY 1040
#define HMC_CTRL_READY_STRIDE 16
#define HMC_CTRL_SOURCE 1296 /* + p * STRIDE: last generation peer p published its source buffer for (pull) */
#define HMC_CTRL_COUNTS 1552 /* + p * STRIDE: last count exchange peer p has written its row for */
#define HMC_CTRL_WORDS 2048

typedef struct hmc_ep_dispatch_args {
  const void* tokens;            /* [num_tokens, hidden] bf16, or expert-major rows when source_of_row is NULL */
  const int32_t* source_of_row;  /* [rows] flat (token * top_k + slot) index of each expert-major row, or NULL */
  const int32_t* expert_of_row;  /* [rows] global expert of each expert-major row */
  const int64_t* dispatch_src_off;    /* [experts] rows, from hmc_route_offsets */
  const int64_t* dispatch_target_off; /* [experts] rows */
  int64_t rows;                  /* tokens * top_k */
  int64_t top_k;
  int64_t hidden;
  int64_t ep;
  int64_t local_experts;
  int64_t capacity_rows;         /* rows each peer's receive buffer can hold */
  void* const* peer_buffers;     /* host array [ep]: receive buffer of every rank, as mapped here */
  void* const* peer_ctrl;        /* host array [ep]: control block of every rank, as mapped here */
  const int32_t* local_ctrl;     /* this rank's own control block */
  int32_t generation;
  int32_t max_ctas;              /* 0 = default */
  uint64_t budget_ns;            /* bound of the ready wait, 0 = 10 s */
  int32_t* status;
  /* Optional scalar per row (the routing probability when probabilities are applied before FC2;
   * reference: probability planes, ops/common/mega_moe/contracts/probability_abi.h:10-19). The value of
   * row j, row_values[value_index ? value_index[j] : j], is stored as float at
   * (char*)peer_buffer + value_plane_offset + 4 * destination_row on the owner. */
  const float* row_values;
  const int32_t* value_index;
  int64_t value_plane_offset;    /* bytes; at least capacity_rows * hidden * 2 */
  int64_t rank;                  /* this rank (0 <= rank < ep); used with send_order_start */
  const int64_t* send_order_start; /* optional device [ep * local_experts + 1], from hmc_route_offsets: when the
                                    dispatch rides inside a grouped GEMM (hmc_grouped_gemm_args.dispatch) the rows
                                    are sent local-expert-major across the destinations (rank + 1 first, this rank
                                    last), so every owner's first experts complete first and their tiles overlap
                                    the rest of the transfer. NULL = source row order */
  const int32_t* skip_flag;      /* optional: as in hmc_grouped_gemm_args */
} hmc_ep_dispatch_args;

typedef struct hmc_ep_combine_args {
  const void* results;               /* [rows, hidden] bf16 in the owner's receive layout */
  const int64_t* segment_start;      /* [local_experts * ep] first row of (local expert, source), buffer order */
  const int64_t* combine_target_off; /* [ep * local_experts] rows, from hmc_route_offsets */
  int64_t rows;
  int64_t hidden;
  int64_t ep;
  int64_t local_experts;
  int64_t target_rows_limit;     /* rows each source's routed buffer can hold */
  void* const* peer_buffers;     /* host array [ep]: routed (combine target) buffer of every rank */
  void* const* peer_ctrl;
  const int32_t* local_ctrl;
  int32_t generation;
  int32_t max_ctas;
  uint64_t budget_ns;
  int32_t* status;
  const float* result_values;    /* optional float[rows] (probability gradients), returned with the rows */
  int64_t value_plane_offset;    /* bytes behind the source's routed buffer; at least target_rows_limit * hidden * 2 */
} hmc_ep_combine_args;

int hmc_symm_alloc(int64_t bytes, void** out); /* cudaMalloc + zero; set-up time only */
int hmc_symm_free(void* ptr);
int hmc_ipc_get_handle(void* ptr, void* handle_out_64_bytes);
int hmc_ipc_open_handle(const void* handle_64_bytes, void** out);
int hmc_ipc_close_handle(void* ptr);
int hmc_ep_publish_ready(void* const* peer_ctrl, int64_t ep, int64_t rank, int32_t generation, void* stream);
int hmc_ep_dispatch(const hmc_ep_dispatch_args* args, void* stream);

/* Pull dispatch: the owner fetches its rows from the sources' published, expert-major source buffers
 * (the reference's pull mode: docs/design/mega_moe_design.md:33-35, transport.h:12-42; the source buffer
 * of hyper_multicore/modules/mega_moe/workspace.py:48-75). A source publishes with
 * hmc_ep_publish_source once its buffer is written; the owner's kernel waits (bounded) for that flag,
 * then copies segment (local expert, source) = source rows [source_row_off[s * local_experts + e], +n)
 * into its own rows starting at segment_start[e * ep + s]. The receive buffer is a plain local
 * allocation of exactly `rows` rows: pull needs no receive capacity in peer-mapped memory. The source
 * may rewrite its buffer once its own result rows are back (every owner has read before it combines). */
typedef struct hmc_ep_pull_args {
  void* const* peer_sources;       /* host array [ep]: source buffer of every rank, as mapped here */
  const int64_t* source_row_off;   /* device [ep * local_experts]: combine_target_off of hmc_route_offsets */
  const int64_t* segment_start;    /* device [local_experts * ep]: recv_segment_start of hmc_route_offsets */
  void* out;                       /* [rows, hidden] bf16, local */
  float* out_values;               /* optional float[rows]: the per-row scalars of the sources */
  int64_t rows;                    /* rows this rank receives */
  int64_t hidden;
  int64_t ep;
  int64_t local_experts;
  int64_t source_rows_limit;       /* rows of every source buffer */
  int64_t value_plane_offset;      /* bytes from a source buffer to its float plane (with out_values) */
  const int32_t* local_ctrl;
  int32_t generation;
  int32_t max_ctas;
  uint64_t budget_ns;
  int32_t* status;
} hmc_ep_pull_args;

/* Count exchange without a host collective (replaces the all_gather of the route header and the
 * per-expert counts, hyper_multicore/modules/mega_moe/route.py:214-245, 850-878): one kernel stores this
 * rank's row {counts[experts], header[4]} into slot `rank` of every peer's table, publishes
 * HMC_CTRL_COUNTS with release semantics and waits (bounded) until every peer's row of this exchange has
 * arrived. A table holds two exchanges (parity = exchange & 1): {int32 counts[ep][experts];
 * int32 header[ep][4]} each, so a fast rank never overwrites rows a slow rank still reads. */
typedef struct hmc_ep_exchange_args {
  const int32_t* counts;      /* device [experts]: this rank's per-expert route counts */
  int32_t header[4];          /* this rank's header words (validity, tokens, autograd, reserved) */
  void* const* peer_tables;   /* host array [ep]: count table of every rank, as mapped here */
  void* const* peer_ctrl;
  const int32_t* local_ctrl;
  int64_t ep;
  int64_t rank;
  int64_t experts;
  int32_t exchange;           /* 1, 2, 3, ...: the same sequence on every rank */
  int32_t reserved;
  uint64_t budget_ns;
  int32_t* status;
} hmc_ep_exchange_args;

int64_t hmc_ep_exchange_table_bytes(int64_t ep, int64_t experts);
int hmc_ep_exchange_counts(const hmc_ep_exchange_args* args, void* stream);
/* Copies `words` int32 from device memory to `dst` with a kernel (plain stores). `dst` may be pinned host
 * memory (device-accessible under unified addressing): small read-backs such as the route counts then do
 * not queue behind bulk device-to-host copies in a copy engine. No counterpart in the reference. */
int hmc_store_words(int32_t* dst, const int32_t* src, int64_t words, void* stream);
/* The same for two sources in one launch: dst[0 .. first_words) = first, then second behind it. */
int hmc_store_words_pair(int32_t* dst, const int32_t* first, int64_t first_words, const int32_t* second,
                         int64_t second_words, void* stream);
int hmc_ep_publish_source(void* const* peer_ctrl, int64_t ep, int64_t rank, int32_t generation, void* stream);
int hmc_ep_pull(const hmc_ep_pull_args* args, void* stream);
int hmc_ep_combine(const hmc_ep_combine_args* args, void* stream);
/* Bounded device-side wait until *counter >= expected; on time-out writes HMC_STATUS_TIMEOUT_ARRIVAL. */
int hmc_ep_wait(const int32_t* counter, int32_t expected, uint64_t budget_ns, int32_t* status, void* stream);
/* The same wait, skipped when *skip_flag is non-zero (skip_flag may be NULL). */
int hmc_ep_wait_groups_unless(const int32_t* counters, const int64_t* group_ends, int64_t groups, uint64_t budget_ns,
                               int32_t* status, const int32_t* skip_flag, void* stream);
int hmc_ep_wait_unless(const int32_t* counter, int32_t expected, uint64_t budget_ns, int32_t* status,
                       const int32_t* skip_flag, void* stream);
/* Admission check of one expert-parallel call ON THE DEVICE, so that the host need not wait for the count table
 * before it queues the operator (the reference reads the table back and validates on the host before every
 * launch, hyper_multicore/modules/mega_moe/route.py:585-622; here the same decision is taken by every rank's
 * device from the same table, and the host validates the mirrored table afterwards, off the critical path).
 * table = {int32 counts[ep][experts]; int32 header[ep][4]} as written by hmc_ep_exchange_counts. *skip_flag is set
 * to 1 when any rank flagged its inputs invalid (header word 0), when any rank would receive more than
 * capacity_rows rows, or when any rank routes more than routed_limit rows; else to 0. Every rank computes the
 * same value, and kernels given the flag do nothing when it is set: nobody stores, nobody waits. The table, the
 * status words (HMC_STATUS_WORDS, may be NULL) and the flag are then copied to host_mirror (pinned host memory,
 * ep * (experts + 4) + HMC_STATUS_WORDS + 1 words) by the kernel itself. */
int hmc_route_guard(const int32_t* table, int64_t ep, int64_t experts, int64_t capacity_rows, int64_t routed_limit,
                    const int32_t* status_words, int32_t* skip_flag, int32_t* host_mirror, void* stream);
/* Bounded device-side wait until counters[g] >= rows of group g for every group (used where a
 * kernel without its own arrival gating consumes dispatched rows, e.g. the MX quantiser). */
int hmc_ep_wait_groups(const int32_t* counters, const int64_t* group_ends, int64_t groups, uint64_t budget_ns,
                       int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * MegaMoE operators: one call per direction, every buffer allocated by the caller.
 * hmc_mega_moe             replaces torch.ops.hyper_multicore.mega_moe
 *                          (hyper_multicore/torch/csrc/registration.cpp:30-60, wrapper torch/ops.py:554-649)
 * hmc_mega_moe_grad        replaces mega_moe_grad (registration.cpp:70-107, torch/ops.py:652-737)
 * hmc_mega_moe_mxfp8(_grad) replace mega_moe_mxfp8 / mega_moe_mxfp8_grad
 *                          (hyper_multicore/torch/csrc/mega_moe_mxfp8.cpp:36-42; buffer order of
 *                          hyper_multicore/modules/mega_moe/backends/mxfp8/execution.py:88-96, 147-155)
 * Each struct lists the reference op's tensors first, under the reference's names and in its order
 * (offsets are in ROWS here, the reference multiplies them by the hidden size), then the fields that
 * stand for what the reference passes as tiling tensors, workspaces and RuntimeConfig blobs (this
 * implementation schedules tiles on the device and needs no host task graph).
 *
 * One call enqueues the whole operator on `stream`: per-call counters cleared and "ready"
 * published, dispatch (push: peer stores issued by extra warps of the first GEMM, so the transfer
 * overlaps its tiles; pull: published source buffer + owner-side fetch; one rank: a local gather),
 * the grouped GEMMs with their fused SwiGLU / SwiGLU-grad epilogues, combine (result rows leave the
 * epilogue of the last row-ragged GEMM for their source ranks), the bounded wait for this rank's own
 * rows, and the owned copies of buffers the next call rewrites. Optional prologue / epilogue fields
 * fold the token-order steps of the reference's autograd function into the same call
 * (restore_topk_output, mega_moe_unpermute_grad_out, moe_token_permute_grad).
 * The first call on a device creates two CUDA events there (used to order the copy stream); make it
 * outside stream capture.
 * ------------------------------------------------------------------------------------------ */
#define HMC_MOE_LAYOUT_EIO 0 /* W1 [e, H, 2I], W2 [e, I, H] */
#define HMC_MOE_LAYOUT_EOI 1 /* W1 [e, 2I, H], W2 [e, H, I] */
#define HMC_MOE_DISPATCH_PUSH 0
#define HMC_MOE_DISPATCH_PULL 1

/* Transport endpoints of one expert-parallel group member (the reference's symmetric workspace,
 * hyper_multicore/modules/mega_moe/workspace.py:48-75, as peer-mapped pointers). */
typedef struct hmc_moe_transport {
  int64_t ep;
  int64_t rank;
  void* const* peer_dispatch;    /* host [ep]: receive buffer of every rank (pull: its published source buffer) */
  void* const* peer_combine;     /* host [ep]: routed buffer of every rank; NULL when ep == 1 */
  void* const* peer_ctrl;        /* host [ep]: control block of every rank (this rank's = all_event_counters) */
  int64_t dispatch_rows_limit;   /* rows every peer_dispatch buffer holds */
  int64_t combine_rows_limit;    /* rows every peer_combine buffer holds */
  int64_t dispatch_plane_offset; /* bytes from a dispatch buffer to its float-per-row plane */
  int64_t combine_plane_offset;  /* bytes from a routed buffer to its float-per-row plane */
  int32_t generation;            /* of this call: grows by one per operator call, the same on every rank */
  int32_t dispatch_mode;         /* HMC_MOE_DISPATCH_* */
  uint64_t wait_budget_ns;       /* bound of every cross-rank device wait, 0 = 10 s */
  void* copy_stream;             /* optional second stream for the owned copies; NULL = on `stream` */
} hmc_moe_transport;

typedef struct hmc_mega_moe_args {
  /* --- the reference op's tensors, in its order --- */
  void* dispatch_target;              /* [>= received_rows, H] bf16: this rank's receive buffer */
  const int64_t* dispatch_target_off; /* [experts] */
  const void* dispatch_src;           /* expert-major rows [routed_rows, H], or the tokens [seq, H] when
                                         dispatch_src_index is given (the permutation is then fused) */
  const int64_t* dispatch_src_off;    /* [experts] */
  const int32_t* dispatch_size;       /* [experts]; not read (sizes follow from the offsets) */
  const void* up_proj_weight;
  const int64_t* up_proj_glist;       /* [experts / ep] cumulative received rows */
  void* up_proj_y;                    /* [rows, 2I] bf16 out */
  void* swiglu_out;                   /* [rows, I] bf16 out */
  const void* down_proj_weight;
  const int64_t* down_proj_glist;     /* the same tensor as up_proj_glist */
  void* down_proj_y;                  /* [rows, H] bf16 out; only written when ep == 1 (with ep > 1 the rows
                                         leave the epilogue for combine_target on their source ranks) */
  void* combine_target;               /* this rank's routed buffer [routed_rows, H]; NULL when ep == 1 */
  const int64_t* combine_target_off;  /* [ep * experts / ep] */
  const int64_t* combine_src_off;     /* not read (recv_segment_start carries the same rows in buffer order) */
  const int32_t* combine_size;        /* not read */
  int32_t* all_event_counters;        /* this rank's control block (HMC_CTRL_WORDS) */
  int32_t* diagnostic_buffer;         /* device status words (HMC_STATUS_WORDS) or NULL */
  int64_t rank_id;
  int64_t ep;
  int64_t expert_num;                 /* global */
  int64_t hidden_size;
  int64_t seq_size;                   /* tokens of this rank */
  /* --- in place of tiling tensors / RuntimeConfig --- */
  int64_t intermediate_size;
  int64_t top_k;
  int64_t routed_rows;                /* seq_size * top_k */
  int64_t received_rows;              /* rows this rank's experts receive */
  int32_t weight_layout;              /* HMC_MOE_LAYOUT_* */
  int32_t swiglu_clamp;               /* HMC_CLAMP_* */
  float swiglu_limit;
  int32_t fuse_dispatch;              /* push with ep > 1: 1 = dispatch warps inside GEMM1 (default choice of the
                                         module), 0 = the stand-alone dispatch kernel first */
  int32_t probs_before_fc2;           /* 1: the routing probabilities travel with the rows and weight the activation
                                         (numerics.py:21-50 apply_probs_before_fc2); the same on every rank */
  int32_t reserved;
  const int32_t* dispatch_src_index;  /* [routed_rows] flat (token * top_k + slot) of each expert-major row, or NULL */
  const int32_t* expert_of_row;       /* [routed_rows] global expert of each expert-major row */
  const int64_t* recv_segment_start;  /* [experts / ep * ep], from hmc_route_offsets */
  const int64_t* send_order_start;    /* [experts + 1], from hmc_route_offsets: order of a GEMM-carried dispatch; or NULL */
  const float* route_probs;           /* [seq * top_k], read with probs_before_fc2 (may be NULL on a rank without tokens) */
  float* row_probs;                   /* before FC2: where the received per-row probabilities are (push: the float
                                         plane of dispatch_target; pull: a caller tensor of received_rows floats) */
  const hmc_moe_transport* transport;
  /* owned copies of what the next call rewrites (ep > 1); each may be NULL */
  void* saved_dispatch;               /* [received_rows, H] <- dispatch_target (push only) */
  void* saved_combine;                /* [routed_rows, H] <- combine_target */
  float* saved_row_probs;             /* [received_rows] <- row_probs (push, before FC2) */
  /* optional epilogue: the weighted Top-K sum back to token order (restore_topk_output,
   * hyper_multicore/modules/mega_moe/route.py:1029-1051) */
  const int32_t* mapping;             /* [seq * top_k] destination row of every (token, slot) */
  const float* topk_probs;            /* [seq * top_k]; not used with route_probs (rows are already weighted) */
  void* output;                       /* [seq, H] bf16, or NULL to skip the epilogue */
  const int32_t* skip_flag;           /* optional, from hmc_route_guard: when set on the device the whole operator is a
                                         no-op there. received_rows may then be an UPPER BOUND (the receive capacity)
                                         instead of the exact count: tiles follow the device-side group list */
} hmc_mega_moe_args;

typedef struct hmc_mega_moe_grad_args {
  /* --- the reference op's tensors, in its order --- */
  void* dispatch_target;              /* [>= received_rows, H]: received dY rows */
  const int64_t* dispatch_target_off;
  const void* dy;                     /* dispatch source: expert-major dY rows [routed_rows, H] (written by the
                                         prologue when grad_output is given), or the token gradients [seq, H]
                                         with dispatch_src_index (probabilities before FC2) */
  const int64_t* dispatch_src_off;
  const int32_t* dispatch_size;       /* not read */
  const void* hidden;                 /* saved swiglu_out [rows, I] */
  void* hidden_dw;                    /* dW2 in the layout of w2, bf16 or f32; NULL = not needed */
  const void* w2;
  void* act_grad_y;                   /* not written: dAct stays in the accumulator of the fused SwiGLU-grad epilogue */
  const void* gate;                   /* saved up_proj_y [rows, 2I] */
  void* grad_gate;                    /* dU [rows, 2I] bf16 out */
  const void* w1;
  void* gate_dx;                      /* dX rows [rows, H]; NULL when they leave the epilogue for grad_x (ep > 1,
                                         probabilities after FC2) */
  void* grad_x;                       /* this rank's routed buffer (combine target); NULL when ep == 1 */
  const int64_t* combine_target_off;
  const int64_t* combine_src_off;     /* not read */
  const int32_t* combine_size;        /* not read */
  const void* permute_out;            /* saved received X rows [rows, H] (for dW1) */
  void* gate_dw;                      /* dW1 in the layout of w1; NULL = not needed */
  const int64_t* group_list;
  int32_t* all_event_counters;
  int32_t* diagnostic_buffer;
  int64_t rank_id;
  int64_t ep;
  int64_t expert_num;
  int64_t hidden_size;
  int64_t seq_size;
  /* --- in place of tiling tensors / RuntimeConfig --- */
  int64_t intermediate_size;
  int64_t top_k;
  int64_t routed_rows;
  int64_t received_rows;
  int32_t weight_layout;
  int32_t swiglu_clamp;
  float swiglu_limit;
  int32_t fuse_dispatch;
  int32_t weight_grad_f32;            /* 1: hidden_dw / gate_dw are FP32 partial gradients (numerics.py:32-34) */
  int32_t probs_before_fc2;           /* as in hmc_mega_moe_args */
  const int32_t* dispatch_src_index;  /* before FC2 only */
  const int32_t* expert_of_row;
  const int64_t* recv_segment_start;
  const int64_t* send_order_start;    /* as in hmc_mega_moe_args */
  const float* row_probs;             /* before FC2: received per-row probabilities saved by forward */
  float* row_dot;                     /* before FC2: scratch float[rows] for the per-row probability gradient */
  const hmc_moe_transport* transport;
  /* optional prologue (probabilities after FC2): dY rows and the probability gradient from the token
   * gradients (mega_moe_unpermute_grad_out, hyper_multicore/torch/csrc/mega_moe_unpermute.cpp:56-65) */
  const void* grad_output;            /* [seq, H] bf16, or NULL */
  const void* saved_combine;          /* routed forward output saved by hmc_mega_moe */
  const int32_t* mapping;
  const float* topk_probs;
  float* grad_probs;                  /* [seq * top_k] out (before FC2: gathered from the returned per-row values) */
  /* optional epilogue: dX[t] = sum of the token's returned rows (moe_token_permute_grad,
   * hyper_multicore/torch/csrc/moe_token_permute_grad.cpp:29-38) */
  void* grad_hidden;                  /* [seq, H] bf16, or NULL */
} hmc_mega_moe_grad_args;

typedef struct hmc_mega_moe_mxfp8_args {
  /* --- the reference's buffer list, in its order (execution.py:88-96) --- */
  void* dispatch_buffer;              /* [>= received_rows, H] bf16 */
  const int64_t* dispatch_target_off;
  const void* source_buffer;          /* tokens [seq, H] with dispatch_src_index, or expert-major rows */
  const int64_t* dispatch_src_off;
  const int32_t* dispatch_size;       /* not read */
  const void* w1_col_data;            /* e4m3 [e, H, 2I] */
  const int64_t* group_list;
  void* up;                           /* [rows, 2I] bf16 out */
  void* a_row;                        /* quantised activation: row data (see `a` for the other planes) */
  const void* w2_col_data;            /* e4m3 [e, I, H] */
  const int64_t* group_list2;         /* the same tensor as group_list */
  void* down;                         /* [rows, H] bf16 out (ep == 1 only) */
  void* routed_buffer;                /* combine target; NULL when ep == 1 */
  const int64_t* combine_target_off;
  const int64_t* combine_src_off;     /* not read */
  const int32_t* combine_size;        /* not read */
  void* x_row;
  void* x_scale;
  void* x_col;                        /* NULL unless a backward follows */
  void* x_col_scale;
  void* a_scale;
  void* a_col;
  void* a_col_scale;
  const void* w1_col_scale;           /* scale-factor ATOMS of W1 (hmc_mx_pack_weight_scale, axis 0) */
  const void* w2_col_scale;           /* scale-factor atoms of W2 */
  int32_t* all_event_counters;
  int32_t* diagnostic_buffer;
  /* --- in place of the launch metadata blob --- */
  int64_t rank_id, ep, expert_num, hidden_size, seq_size, intermediate_size, top_k, routed_rows, received_rows;
  int64_t pad_blocks;                 /* 128-row blocks the quantised buffers hold (>= ceil(rows/128) + groups) */
  const int32_t* dispatch_src_index;
  const int32_t* expert_of_row;
  const int64_t* recv_segment_start;
  const hmc_moe_transport* transport;
  void* saved_combine;                /* [routed_rows, H] <- routed_buffer (ep > 1) */
  const int32_t* mapping;             /* optional epilogue as in hmc_mega_moe_args */
  const float* topk_probs;
  void* output;
  const int32_t* skip_flag;           /* as in hmc_mega_moe_args: the device-side admission decision of hmc_route_guard */
} hmc_mega_moe_mxfp8_args;

typedef struct hmc_mega_moe_mxfp8_grad_args {
  /* --- the reference's buffer list, in its order (execution.py:147-155) --- */
  void* dispatch;                     /* [>= received_rows, H] bf16: received dY rows */
  const int64_t* dispatch_target_off;
  void* source;                       /* [routed_rows, H] bf16 expert-major dY rows (written by the prologue) */
  const int64_t* dispatch_src_off;
  const int32_t* dispatch_size;       /* not read */
  const void* a_col;                  /* saved by forward */
  void* dw2;                          /* [e, I, H] bf16 or f32; NULL = not needed */
  const void* w2_row_data;            /* e4m3 [e, I, H], blocks along H */
  void* da;                           /* [rows, I] bf16 out */
  const void* up;                     /* saved by forward */
  void* du_row;
  const void* w1_row_data;            /* e4m3 [e, H, 2I], blocks along 2I */
  void* dx;                           /* [rows, H] bf16 out (ep == 1 only) */
  void* routed_buffer;                /* combine target; NULL when ep == 1 */
  const int64_t* combine_target_off;
  const int64_t* combine_src_off;     /* not read */
  const int32_t* combine_size;        /* not read */
  const void* x_col;                  /* saved by forward */
  void* dw1;                          /* [e, H, 2I]; NULL = not needed */
  const int64_t* group_list;
  void* dy_row;
  void* dy_scale;
  void* dy_col;
  void* dy_col_scale;
  const void* a_col_scale;
  const void* w2_row_scale;           /* scale-factor atoms (hmc_mx_pack_weight_scale, axis 1) */
  void* du_scale;
  void* du_col;
  void* du_col_scale;
  const void* w1_row_scale;           /* scale-factor atoms */
  const void* x_col_scale;
  int32_t* all_event_counters;
  int32_t* diagnostic_buffer;
  /* --- in place of the launch metadata blob --- */
  int64_t rank_id, ep, expert_num, hidden_size, seq_size, intermediate_size, top_k, routed_rows, received_rows;
  int64_t pad_blocks;
  int32_t weight_grad_f32;
  int32_t reserved;
  const int64_t* recv_segment_start;
  const int32_t* expert_of_row;
  const hmc_moe_transport* transport;
  /* prologue / epilogue as in hmc_mega_moe_grad_args */
  const void* grad_output;
  const void* saved_combine;
  const int32_t* mapping;
  const float* topk_probs;
  float* grad_probs;
  void* grad_hidden;
  const int32_t* skip_flag;
} hmc_mega_moe_mxfp8_grad_args;

int hmc_mega_moe(const hmc_mega_moe_args* args, void* stream);
int hmc_mega_moe_grad(const hmc_mega_moe_grad_args* args, void* stream);
int hmc_mega_moe_mxfp8(const hmc_mega_moe_mxfp8_args* args, void* stream);
int hmc_mega_moe_mxfp8_grad(const hmc_mega_moe_mxfp8_grad_args* args, void* stream);
/* ABI version of the MXFP8 operator pair the reference's loader asserts (mega_moe_mxfp8.cpp: == 3). */
int hmc_mega_moe_mxfp8_abi_version(void);

#ifdef __cplusplus
}
#endif

#endif /* HMC_B200_H_ */
