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
#define HMC_EPI_STORE_BF16 0
#define HMC_EPI_STORE_F32 1   /* RAGGED_K only: FP32 partial weight gradients */
#define HMC_EPI_SWIGLU 2      /* B has 2n columns [gate | up]; c = U[rows, 2n], aux = Act[rows, n] */
#define HMC_EPI_SWIGLU_GRAD 3 /* acc = dAct[rows, n]; aux = U[rows, 2n] (input); c = dU[rows, 2n] */

typedef struct hmc_grouped_gemm_args {
  int32_t mode;
  int32_t a_major; /* RAGGED_M: HMC_MAJOR_K. RAGGED_K: HMC_MAJOR_MN */
  int32_t b_major; /* RAGGED_M: MN = B[groups, k, n_cols], K = B[groups, n_cols, k] */
  int32_t epilogue;
  int32_t groups;
  int32_t max_ctas; /* 0 = one CTA per SM */
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
} hmc_grouped_gemm_args;

int hmc_grouped_gemm(const hmc_grouped_gemm_args* args, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* HMC_B200_H_ */
