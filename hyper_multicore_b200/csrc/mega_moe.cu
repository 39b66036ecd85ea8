// Operator-level entry points of the MegaMoE path: one call per direction issues the whole launch
// sequence on the caller's stream.
//
// Replaces torch.ops.hyper_multicore.mega_moe / mega_moe_grad (hyper_multicore/torch/csrc/
// registration.cpp:30-107) and mega_moe_mxfp8 / mega_moe_mxfp8_grad (torch/csrc/mega_moe_mxfp8.cpp:36-42).
// The reference hands its device megakernel a host-built task graph (tasks/gmm.py, tasks/alltoall.py,
// backends/bf16/forward/graph.py:100-172, backward/graph.py:121-259, backends/mxfp8/graph.py:116-180);
// here the same stages are a fixed sequence of launches whose tiles are scheduled on the device:
//   forward : counters cleared + ready published -> dispatch (inside GEMM1) -> GEMM1 + SwiGLU
//             -> GEMM2 (+ combine from its epilogue) -> bounded wait for the returned rows -> Top-K sum
//   backward: dY rows + dProbs -> dispatch (inside the dA GEMM) -> dA + SwiGLU-grad -> dX (+ combine)
//             -> dW2, dW1 -> bounded wait -> Top-K sum of dX
#include <string.h>

#include <stdlib.h>

#include "common.cuh"

namespace hmc {
namespace {

// dst[i] = src[index[i]] for floats (per-row probabilities into expert-major order and back).
__global__ void gather_floats_kernel(float* __restrict__ dst, const float* __restrict__ src,
                                     const int* __restrict__ index, long long n, long long src_n, int* status) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long j = index[i];
    if (j < 0 || j >= src_n) {
      report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(i), static_cast<int>(j), 0);
      dst[i] = 0.0f;
    } else {
      dst[i] = src[j];
    }
  }
}

int gather_floats(float* dst, const float* src, const int* index, long long n, long long src_n, int* status,
                  cudaStream_t stream) {
  if (n == 0) return 0;
  const int blocks = static_cast<int>(n < 256ll * 1024 ? (n + 255) / 256 : 1024);
  gather_floats_kernel<<<blocks, 256, 0, stream>>>(dst, src, index, n, src_n, status);
  HMC_LAUNCH_OK();
  return 0;
}

// Two events per device order the optional copy stream against the operator's stream.
struct CopyEvents {
  cudaEvent_t fork;
  cudaEvent_t join;
};

int copy_events(CopyEvents** out) {
  static CopyEvents events[HMC_MAX_DEVICES];
  static bool created[HMC_MAX_DEVICES];
  int dev = 0;
  HMC_CUDA_OK(cudaGetDevice(&dev));
  HMC_REQUIRE(dev >= 0 && dev < HMC_MAX_DEVICES, HMC_ERR_LIMIT, "device ordinal %d not supported", dev);
  if (!created[dev]) {
    HMC_CUDA_OK(cudaEventCreateWithFlags(&events[dev].fork, cudaEventDisableTiming));
    HMC_CUDA_OK(cudaEventCreateWithFlags(&events[dev].join, cudaEventDisableTiming));
    created[dev] = true;
  }
  *out = &events[dev];
  return 0;
}

// Runs owned copies beside the operator's own kernels: `begin` makes the copy stream wait for the work
// queued so far, `copy` enqueues device-to-device copies there, `end` makes the operator's stream wait
// for them. Without a copy stream everything stays on the operator's stream.
struct SideCopies {
  cudaStream_t main;
  cudaStream_t side;
  CopyEvents* events;
  bool open;

  int init(cudaStream_t main_stream, void* copy_stream) {
    main = main_stream;
    side = static_cast<cudaStream_t>(copy_stream);
    events = nullptr;
    open = false;
    if (side != nullptr && side != main) return copy_events(&events);
    side = main;
    return 0;
  }
  int begin() {
    if (side != main) {
      HMC_CUDA_OK(cudaEventRecord(events->fork, main));
      HMC_CUDA_OK(cudaStreamWaitEvent(side, events->fork, 0));
      open = true;
    }
    return 0;
  }
  int copy(void* dst, const void* src, size_t bytes) {
    if (bytes == 0 || dst == nullptr || dst == src) return 0;
    HMC_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, side));
    return 0;
  }
  int end() {
    if (open) {
      HMC_CUDA_OK(cudaEventRecord(events->join, side));
      HMC_CUDA_OK(cudaStreamWaitEvent(main, events->join, 0));
      open = false;
    }
    return 0;
  }
};

#define HMC_TRY(expr)          \
  do {                         \
    int rc__ = (expr);         \
    if (rc__ != 0) return rc__; \
  } while (0)

int check_transport(const hmc_moe_transport* t, const char* who, int64_t ep, int64_t rank, const void* ctrl,
                    bool need_combine) {
  HMC_REQUIRE(t != nullptr, HMC_ERR_INVALID, "%s: null transport", who);
  HMC_REQUIRE(t->ep == ep && t->rank == rank && ep >= 1 && ep <= HMC_MAX_EP && rank >= 0 && rank < ep,
              HMC_ERR_INVALID, "%s: transport ep / rank (%lld, %lld) do not match the operator's (%lld, %lld)", who,
              (long long)t->ep, (long long)t->rank, (long long)ep, (long long)rank);
  HMC_REQUIRE(t->peer_ctrl != nullptr && t->peer_ctrl[rank] == ctrl, HMC_ERR_INVALID,
              "%s: all_event_counters must be this rank's entry of transport.peer_ctrl", who);
  HMC_REQUIRE(t->dispatch_mode == HMC_MOE_DISPATCH_PUSH || t->dispatch_mode == HMC_MOE_DISPATCH_PULL, HMC_ERR_INVALID,
              "%s: unknown dispatch mode %d", who, t->dispatch_mode);
  HMC_REQUIRE(!need_combine || t->peer_combine != nullptr, HMC_ERR_INVALID,
              "%s: expert parallelism needs the peers' routed buffers", who);
  return 0;
}

// Per-call counters cleared on the stream, then "this rank's buffers are free for generation g" published.
int begin_call(const hmc_moe_transport& t, int32_t* ctrl, cudaStream_t stream) {
  HMC_CUDA_OK(cudaMemsetAsync(ctrl, 0, sizeof(int32_t) * HMC_CTRL_READY, stream));
  return hmc_ep_publish_ready(t.peer_ctrl, t.ep, t.rank, t.generation, stream);
}

struct Shape {
  int64_t hidden, inter, top_k, local, routed, received, rows, tokens;
};

hmc_gemm_combine make_combine(const hmc_moe_transport& t, const int64_t* segment_start, const int64_t* target_off,
                              int64_t local) {
  hmc_gemm_combine c;
  memset(&c, 0, sizeof(c));
  c.segment_start = segment_start;
  c.combine_target_off = target_off;
  c.peer_buffers = t.peer_combine;
  c.peer_ctrl = t.peer_ctrl;
  c.ep = t.ep;
  c.local_experts = local;
  c.target_rows_limit = t.combine_rows_limit;
  return c;
}

hmc_ep_dispatch_args make_dispatch(const hmc_moe_transport& t, const void* src, const int32_t* src_index,
                                   const int32_t* expert_of_row, const int64_t* src_off, const int64_t* target_off,
                                   const Shape& s, int32_t* ctrl, int32_t* status, const int64_t* send_order = nullptr,
                                   const int32_t* skip_flag = nullptr) {
  hmc_ep_dispatch_args d;
  memset(&d, 0, sizeof(d));
  d.tokens = src;
  d.source_of_row = src_index;
  d.expert_of_row = expert_of_row;
  d.dispatch_src_off = src_off;
  d.dispatch_target_off = target_off;
  d.rows = s.routed;
  d.top_k = s.top_k;
  d.hidden = s.hidden;
  d.ep = t.ep;
  d.local_experts = s.local;
  d.capacity_rows = t.dispatch_rows_limit;
  d.peer_buffers = t.peer_dispatch;
  d.peer_ctrl = t.peer_ctrl;
  d.local_ctrl = ctrl;
  d.generation = t.generation;
  d.budget_ns = t.wait_budget_ns;
  d.status = status;
  d.rank = t.rank;
  d.send_order_start = send_order;
  d.skip_flag = skip_flag;
  return d;
}

// Pull dispatch: this rank's expert-major rows go into its published source buffer, then the owner side
// fetches the rows of its own experts from every source (docs/design/mega_moe_design.md:33-35).
// `fill` has already written the source buffer when it is the caller's job (backward prologue).
int pull_rows(const hmc_moe_transport& t, const Shape& s, const int64_t* recv_segment_start,
              const int64_t* combine_target_off, void* out, float* out_values, int32_t* ctrl, int32_t* status,
              cudaStream_t stream) {
  HMC_TRY(hmc_ep_publish_source(t.peer_ctrl, t.ep, t.rank, t.generation, stream));
  hmc_ep_pull_args p;
  memset(&p, 0, sizeof(p));
  p.peer_sources = t.peer_dispatch;
  p.source_row_off = combine_target_off;
  p.segment_start = recv_segment_start;
  p.out = out;
  p.out_values = out_values;
  p.rows = s.received;
  p.hidden = s.hidden;
  p.ep = t.ep;
  p.local_experts = s.local;
  p.source_rows_limit = t.dispatch_rows_limit;
  p.value_plane_offset = t.dispatch_plane_offset;
  p.local_ctrl = ctrl;
  p.generation = t.generation;
  p.budget_ns = t.wait_budget_ns;
  p.status = status;
  return hmc_ep_pull(&p, stream);
}

hmc_grouped_gemm_args ragged_m(const void* a, const void* b, void* c, const int64_t* group_ends, const Shape& s,
                               int64_t n, int64_t k, int b_major, int epilogue, int32_t* status) {
  hmc_grouped_gemm_args g;
  memset(&g, 0, sizeof(g));
  g.mode = HMC_GEMM_RAGGED_M;
  g.a_major = HMC_MAJOR_K;
  g.b_major = b_major;
  g.epilogue = epilogue;
  g.groups = static_cast<int32_t>(s.local);
  g.rows = s.received;
  g.n = n;
  g.k = k;
  g.a = a;
  g.b = b;
  g.c = c;
  g.group_ends = group_ends;
  g.status = status;
  return g;
}

hmc_grouped_gemm_args ragged_k(const void* a, const void* b, void* c, const int64_t* group_ends, const Shape& s,
                               int64_t m, int64_t n, bool f32, int32_t* status) {
  hmc_grouped_gemm_args g;
  memset(&g, 0, sizeof(g));
  g.mode = HMC_GEMM_RAGGED_K;
  g.a_major = HMC_MAJOR_MN;
  g.b_major = HMC_MAJOR_MN;
  g.epilogue = f32 ? HMC_EPI_STORE_F32 : HMC_EPI_STORE_BF16;
  g.groups = static_cast<int32_t>(s.local);
  g.rows = s.received;
  g.m = m;
  g.n = n;
  g.a = a;
  g.b = b;
  g.c = c;
  g.group_ends = group_ends;
  g.status = status;
  return g;
}

int check_shape(const char* who, int64_t ep, int64_t rank, int64_t experts, int64_t hidden, int64_t inter, int64_t tokens,
                int64_t top_k, int64_t routed, int64_t received, Shape* s) {
  HMC_REQUIRE(ep >= 1 && ep <= HMC_MAX_EP && rank >= 0 && rank < ep, HMC_ERR_INVALID, "%s: bad ep / rank", who);
  HMC_REQUIRE(experts > 0 && experts % ep == 0 && experts / ep <= HMC_CTRL_MAX_LOCAL_EXPERTS, HMC_ERR_INVALID,
              "%s: expert_num (%lld) must be a positive multiple of ep (%lld)", who, (long long)experts, (long long)ep);
  HMC_REQUIRE(hidden > 0 && hidden % 8 == 0 && inter > 0 && inter % 8 == 0, HMC_ERR_INVALID,
              "%s: hidden (%lld) and intermediate (%lld) sizes must be positive multiples of 8", who, (long long)hidden,
              (long long)inter);
  HMC_REQUIRE(tokens >= 0 && top_k > 0 && routed == tokens * top_k && received >= 0 && routed < (1ll << 31) &&
                  received < (1ll << 31),
              HMC_ERR_INVALID, "%s: routed_rows must equal seq_size * top_k and row counts must fit in int32", who);
  s->hidden = hidden;
  s->inter = inter;
  s->top_k = top_k;
  s->local = experts / ep;
  s->routed = routed;
  s->received = received;
  s->rows = received > 0 ? received : 1;
  s->tokens = tokens;
  return 0;
}

}  // namespace
}  // namespace hmc

using namespace hmc;

extern "C" int hmc_mega_moe_mxfp8_abi_version(void) { return 3; }

// ================================================================================================ BF16 forward
extern "C" int hmc_mega_moe(const hmc_mega_moe_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mega_moe: null args");
  const hmc_mega_moe_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  Shape s;
  HMC_TRY(check_shape("hmc_mega_moe", a.ep, a.rank_id, a.expert_num, a.hidden_size, a.intermediate_size, a.seq_size,
                      a.top_k, a.routed_rows, a.received_rows, &s));
  HMC_REQUIRE(a.dispatch_target && (a.dispatch_src || a.routed_rows == 0) && a.up_proj_weight && a.up_proj_glist &&
                  a.up_proj_y && a.swiglu_out && a.down_proj_weight && a.all_event_counters,
              HMC_ERR_INVALID, "hmc_mega_moe: null tensor pointer");
  HMC_REQUIRE(a.down_proj_glist == nullptr || a.down_proj_glist == a.up_proj_glist, HMC_ERR_INVALID,
              "hmc_mega_moe: both GEMMs walk the same group list");
  HMC_REQUIRE(a.weight_layout == HMC_MOE_LAYOUT_EIO || a.weight_layout == HMC_MOE_LAYOUT_EOI, HMC_ERR_INVALID,
              "hmc_mega_moe: unknown weight layout %d", a.weight_layout);
  const bool ep1 = a.ep == 1;
  HMC_TRY(check_transport(a.transport, "hmc_mega_moe", a.ep, a.rank_id, a.all_event_counters, !ep1));
  const hmc_moe_transport& t = *a.transport;
  const bool before_fc2 = a.probs_before_fc2 != 0;
  const bool pull = !ep1 && t.dispatch_mode == HMC_MOE_DISPATCH_PULL;
  const bool local_gather = ep1 && !before_fc2;  // one rank owns every expert: a gather, nothing to wait for
  HMC_REQUIRE(ep1 ? a.down_proj_y != nullptr : a.combine_target != nullptr, HMC_ERR_INVALID,
              "hmc_mega_moe: down_proj_y (one rank) or combine_target (expert parallel) is required");
  HMC_REQUIRE(local_gather || ((a.expert_of_row || s.routed == 0) && a.dispatch_src_off && a.dispatch_target_off),
              HMC_ERR_INVALID,
              "hmc_mega_moe: dispatch needs expert_of_row and the dispatch offsets");
  HMC_REQUIRE(ep1 || (a.recv_segment_start && a.combine_target_off), HMC_ERR_INVALID,
              "hmc_mega_moe: combine needs recv_segment_start and combine_target_off");
  HMC_REQUIRE(!before_fc2 || (a.row_probs != nullptr && ((a.dispatch_src_index && a.route_probs) || s.routed == 0)),
              HMC_ERR_INVALID, "hmc_mega_moe: probabilities before FC2 need row_probs for the received rows and dispatch_src_index");
  HMC_REQUIRE(!local_gather || a.dispatch_src_index != nullptr || a.dispatch_src == a.dispatch_target || s.routed == 0,
              HMC_ERR_INVALID,
              "hmc_mega_moe: a single rank gathers its rows through dispatch_src_index");
  HMC_REQUIRE(a.output == nullptr || (a.mapping != nullptr && (before_fc2 || a.topk_probs != nullptr)), HMC_ERR_INVALID,
              "hmc_mega_moe: the Top-K sum needs mapping and topk_probs");
  int32_t* ctrl = a.all_event_counters;
  int32_t* status = a.diagnostic_buffer;
  const int b_major = a.weight_layout == HMC_MOE_LAYOUT_EIO ? HMC_MAJOR_MN : HMC_MAJOR_K;
  SideCopies copies;
  HMC_TRY(copies.init(stream, t.copy_stream));

  const int32_t* arrival = nullptr;
  const float* row_probs = before_fc2 ? a.row_probs : nullptr;
  hmc_ep_dispatch_args dispatch;
  bool fused_dispatch = false;
  if (local_gather) {
    if (s.routed > 0 && a.dispatch_src_index != nullptr)
      HMC_TRY(hmc_moe_gather_rows(a.dispatch_src, a.dispatch_src_index, s.routed, s.top_k, s.hidden, a.dispatch_target,
                                  stream));
  } else {
    HMC_TRY(begin_call(t, ctrl, stream));
    if (pull) {
      // this rank's rows, expert-major, into its own published source buffer
      void* source = t.peer_dispatch[t.rank];
      if (s.routed > 0) {
        if (a.dispatch_src_index != nullptr)
          HMC_TRY(hmc_moe_gather_rows(a.dispatch_src, a.dispatch_src_index, s.routed, s.top_k, s.hidden, source, stream));
        else if (a.dispatch_src != source)
          HMC_CUDA_OK(cudaMemcpyAsync(source, a.dispatch_src, static_cast<size_t>(s.routed) * s.hidden * 2,
                                      cudaMemcpyDeviceToDevice, stream));
        if (before_fc2) {
          float* plane = reinterpret_cast<float*>(static_cast<unsigned char*>(source) + t.dispatch_plane_offset);
          HMC_TRY(gather_floats(plane, a.route_probs, a.dispatch_src_index, s.routed, s.routed, status, stream));
        }
      }
      HMC_TRY(pull_rows(t, s, a.recv_segment_start, a.combine_target_off, a.dispatch_target,
                        before_fc2 ? a.row_probs : nullptr, ctrl, status, stream));
    } else {
      dispatch = make_dispatch(t, a.dispatch_src, a.dispatch_src_index, a.expert_of_row, a.dispatch_src_off,
                               a.dispatch_target_off, s, ctrl, status, a.send_order_start, a.skip_flag);
      if (before_fc2) {
        dispatch.row_values = a.route_probs;
        dispatch.value_index = a.dispatch_src_index;
        dispatch.value_plane_offset = t.dispatch_plane_offset;
      }
      HMC_REQUIRE(t.peer_dispatch[t.rank] == a.dispatch_target, HMC_ERR_INVALID,
                  "hmc_mega_moe: dispatch_target must be this rank's entry of transport.peer_dispatch");
      fused_dispatch = a.fuse_dispatch != 0;
      if (!fused_dispatch) HMC_TRY(hmc_ep_dispatch(&dispatch, stream));
      arrival = ctrl + HMC_CTRL_ARRIVAL;
    }
  }

  // GEMM1 + SwiGLU, gated per expert on the arrival counters when rows come from peers
  if (s.received > 0 || (fused_dispatch && s.routed > 0)) {
    hmc_grouped_gemm_args g = ragged_m(a.dispatch_target, a.up_proj_weight, a.up_proj_y, a.up_proj_glist, s, s.inter,
                                       s.hidden, b_major, HMC_EPI_SWIGLU, status);
    g.aux = a.swiglu_out;
    g.ready_counters = arrival;
    g.ready_budget_ns = t.wait_budget_ns;
    g.swiglu_clamp = a.swiglu_clamp;
    g.swiglu_limit = a.swiglu_limit;
    g.row_probs = row_probs;
    g.dispatch = fused_dispatch ? &dispatch : nullptr;
    g.skip_flag = a.skip_flag;
    HMC_TRY(hmc_grouped_gemm(&g, stream));
  }
  if (!ep1 && !pull && a.saved_dispatch != nullptr && s.received > 0) {
    // GEMM1 has waited for every expert's rows: the owned copy of the received rows (the peer-mapped
    // buffer is rewritten by the next call) runs beside GEMM2.
    HMC_TRY(copies.begin());
    HMC_TRY(copies.copy(a.saved_dispatch, a.dispatch_target, static_cast<size_t>(s.received) * s.hidden * 2));
  }
  hmc_gemm_combine combine;
  if (s.received > 0) {
    hmc_grouped_gemm_args g = ragged_m(a.swiglu_out, a.down_proj_weight, ep1 ? a.down_proj_y : nullptr, a.up_proj_glist, s,
                                       s.hidden, s.inter, b_major, HMC_EPI_STORE_BF16, status);
    if (!ep1) {
      combine = make_combine(t, a.recv_segment_start, a.combine_target_off, s.local);
      g.combine = &combine;
    }
    g.skip_flag = a.skip_flag;
    HMC_TRY(hmc_grouped_gemm(&g, stream));
  }
  const void* routed_rows_ptr = a.down_proj_y;
  if (!ep1) {
    // the result rows left the GEMM2 epilogue for their sources; wait for this rank's own
    HMC_TRY(hmc_ep_wait_unless(ctrl + HMC_CTRL_COMBINE,
                               static_cast<int32_t>(s.routed * hmc_grouped_gemm_combine_units(s.hidden)),
                               t.wait_budget_ns, status, a.skip_flag, stream));
    routed_rows_ptr = a.combine_target;
    if (a.saved_combine != nullptr || (before_fc2 && !pull && a.saved_row_probs != nullptr)) {
      HMC_TRY(copies.begin());
      // (a call that does not fit the workspace is a no-op on the device: copy no more than the buffer holds)
      const int64_t held = s.routed < t.combine_rows_limit ? s.routed : t.combine_rows_limit;
      HMC_TRY(copies.copy(a.saved_combine, a.combine_target, static_cast<size_t>(held) * s.hidden * 2));
      if (before_fc2 && !pull)
        HMC_TRY(copies.copy(a.saved_row_probs, a.row_probs, static_cast<size_t>(s.received) * sizeof(float)));
    }
  }
  if (a.output != nullptr && s.tokens > 0) {
    // before FC2 the rows are already weighted: summed as they are (backends/bf16/autograd.py:133-135)
    const int64_t available = ep1 ? s.rows : t.combine_rows_limit;
    HMC_TRY(moe_unpermute_unless(routed_rows_ptr, a.mapping, before_fc2 ? nullptr : a.topk_probs, s.tokens, s.top_k,
                                 s.hidden, available, a.output, status, a.skip_flag, stream));
  }
  return copies.end();
}

// ================================================================================================ BF16 backward
extern "C" int hmc_mega_moe_grad(const hmc_mega_moe_grad_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_grad: null args");
  const hmc_mega_moe_grad_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  Shape s;
  HMC_TRY(check_shape("hmc_mega_moe_grad", a.ep, a.rank_id, a.expert_num, a.hidden_size, a.intermediate_size, a.seq_size,
                      a.top_k, a.routed_rows, a.received_rows, &s));
  HMC_REQUIRE((a.dy || a.routed_rows == 0) && a.hidden && a.w2 && a.gate && a.grad_gate && a.w1 && a.group_list &&
                  a.all_event_counters,
              HMC_ERR_INVALID, "hmc_mega_moe_grad: null tensor pointer");
  HMC_REQUIRE(a.weight_layout == HMC_MOE_LAYOUT_EIO || a.weight_layout == HMC_MOE_LAYOUT_EOI, HMC_ERR_INVALID,
              "hmc_mega_moe_grad: unknown weight layout %d", a.weight_layout);
  const bool ep1 = a.ep == 1;
  HMC_TRY(check_transport(a.transport, "hmc_mega_moe_grad", a.ep, a.rank_id, a.all_event_counters, !ep1));
  const hmc_moe_transport& t = *a.transport;
  const bool before_fc2 = a.probs_before_fc2 != 0;
  const bool pull = !ep1 && t.dispatch_mode == HMC_MOE_DISPATCH_PULL;
  const bool eio = a.weight_layout == HMC_MOE_LAYOUT_EIO;
  HMC_REQUIRE(!before_fc2 || (a.row_dot != nullptr && a.row_probs != nullptr && (a.dispatch_src_index != nullptr || s.routed == 0)),
              HMC_ERR_INVALID,
              "hmc_mega_moe_grad: probabilities before FC2 need row_dot scratch and dispatch_src_index");
  HMC_REQUIRE(before_fc2 || a.grad_output == nullptr || s.tokens == 0 ||
                  (a.mapping && a.topk_probs && a.grad_probs && a.saved_combine),
              HMC_ERR_INVALID, "hmc_mega_moe_grad: the prologue needs mapping, topk_probs, grad_probs and saved_combine");
  HMC_REQUIRE(a.grad_hidden == nullptr || a.mapping != nullptr || s.tokens == 0, HMC_ERR_INVALID,
              "hmc_mega_moe_grad: the Top-K sum of dX needs mapping");
  HMC_REQUIRE(ep1 || (a.grad_x && a.recv_segment_start && a.combine_target_off && (a.expert_of_row || s.routed == 0)),
              HMC_ERR_INVALID,
              "hmc_mega_moe_grad: expert parallelism needs grad_x, the combine tables and expert_of_row");
  const bool fused_combine = !ep1 && !before_fc2;  // with the probability gradient travelling back the rows
                                                   // return through the combine kernel, which carries it
  HMC_REQUIRE(fused_combine || a.gate_dx != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_grad: gate_dx is required here");
  int32_t* ctrl = a.all_event_counters;
  int32_t* status = a.diagnostic_buffer;
  // Transposed use of the weights: EIO W2 [e, I, H] is the K-major B of dA = dY . W2^T; EOI the reverse.
  const int bt_major = eio ? HMC_MAJOR_K : HMC_MAJOR_MN;

  const void* dy_recv = a.dispatch_target;
  const int32_t* arrival = nullptr;
  hmc_ep_dispatch_args dispatch;
  bool fused_dispatch = false;
  if (before_fc2) {
    // dY rows are plain copies of the token gradients (backends/bf16/autograd.py:138-150): the gather is
    // fused into the dispatch. a.dy holds the token gradients.
    HMC_REQUIRE(a.dispatch_target != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_grad: dispatch_target is required");
    HMC_TRY(begin_call(t, ctrl, stream));
    if (pull) {
      void* source = t.peer_dispatch[t.rank];
      if (s.routed > 0)
        HMC_TRY(hmc_moe_gather_rows(a.dy, a.dispatch_src_index, s.routed, s.top_k, s.hidden, source, stream));
      HMC_TRY(pull_rows(t, s, a.recv_segment_start, a.combine_target_off, a.dispatch_target, nullptr, ctrl, status, stream));
    } else {
      dispatch = make_dispatch(t, a.dy, a.dispatch_src_index, a.expert_of_row, a.dispatch_src_off, a.dispatch_target_off,
                               s, ctrl, status, a.send_order_start);
      HMC_REQUIRE(t.peer_dispatch[t.rank] == a.dispatch_target, HMC_ERR_INVALID,
                  "hmc_mega_moe_grad: dispatch_target must be this rank's entry of transport.peer_dispatch");
      fused_dispatch = a.fuse_dispatch != 0;
      if (!fused_dispatch) HMC_TRY(hmc_ep_dispatch(&dispatch, stream));
      arrival = ctrl + HMC_CTRL_ARRIVAL;
    }
    HMC_CUDA_OK(cudaMemsetAsync(a.row_dot, 0, sizeof(float) * s.rows, stream));
  } else {
    // prologue: dY rows (source's expert-major order) and dProbs from the token gradients
    void* dy_rows = const_cast<void*>(a.dy);
    if (pull) dy_rows = t.peer_dispatch[t.rank];  // written straight into the published source buffer
    if (pull) HMC_TRY(begin_call(t, ctrl, stream));
    if (a.grad_output != nullptr && s.tokens > 0)
      HMC_TRY(hmc_moe_unpermute_grad(a.saved_combine, a.grad_output, a.mapping, a.topk_probs, s.tokens, s.top_k, s.hidden,
                                     dy_rows, a.grad_probs, status, stream));
    if (pull) {
      HMC_REQUIRE(a.dispatch_target != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_grad: dispatch_target is required");
      HMC_TRY(pull_rows(t, s, a.recv_segment_start, a.combine_target_off, a.dispatch_target, nullptr, ctrl, status, stream));
    } else if (ep1) {
      // one rank owns every expert: the source's expert-major order IS the owner's order, the rows are
      // used in place and nothing has to arrive (the reference short-circuits peer == self, rma.h:205-208)
      dy_recv = a.dy;
    } else {
      HMC_REQUIRE(a.dispatch_target != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_grad: dispatch_target is required");
      HMC_TRY(begin_call(t, ctrl, stream));
      dispatch = make_dispatch(t, a.dy, nullptr, a.expert_of_row, a.dispatch_src_off, a.dispatch_target_off, s, ctrl,
                               status, a.send_order_start);
      HMC_REQUIRE(t.peer_dispatch[t.rank] == a.dispatch_target, HMC_ERR_INVALID,
                  "hmc_mega_moe_grad: dispatch_target must be this rank's entry of transport.peer_dispatch");
      fused_dispatch = a.fuse_dispatch != 0;
      if (!fused_dispatch) HMC_TRY(hmc_ep_dispatch(&dispatch, stream));
      arrival = ctrl + HMC_CTRL_ARRIVAL;
    }
  }

  hmc_gemm_combine combine;
  if (s.received > 0 || (fused_dispatch && s.routed > 0)) {
    // dA = dY . W2^T with the SwiGLU gradient in the epilogue: dU = SwiGLU'(dA, U)
    hmc_grouped_gemm_args g = ragged_m(dy_recv, a.w2, a.grad_gate, a.group_list, s, s.inter, s.hidden, bt_major,
                                       HMC_EPI_SWIGLU_GRAD, status);
    g.aux = const_cast<void*>(a.gate);
    g.ready_counters = arrival;
    g.ready_budget_ns = t.wait_budget_ns;
    g.swiglu_clamp = a.swiglu_clamp;
    g.swiglu_limit = a.swiglu_limit;
    g.row_probs = a.row_probs;
    g.row_dot = before_fc2 ? a.row_dot : nullptr;
    g.dispatch = fused_dispatch ? &dispatch : nullptr;
    HMC_TRY(hmc_grouped_gemm(&g, stream));
  }
  if (s.received > 0) {
    // dX rows = dU . W1^T; with expert parallelism they leave the epilogue for their source ranks
    hmc_grouped_gemm_args g = ragged_m(a.grad_gate, a.w1, fused_combine ? nullptr : a.gate_dx, a.group_list, s, s.hidden,
                                       2 * s.inter, bt_major, HMC_EPI_STORE_BF16, status);
    if (fused_combine) {
      combine = make_combine(t, a.recv_segment_start, a.combine_target_off, s.local);
      g.combine = &combine;
    }
    HMC_TRY(hmc_grouped_gemm(&g, stream));
  }
  // Weight gradients (contraction over each expert's rows; cold experts get exact zeros). The arrival wait
  // of the dA GEMM above orders these kernels after the rows have landed. With probabilities before FC2,
  // `hidden` is the weighted activation FC2 actually saw.
  if (a.hidden_dw != nullptr) {
    const void* x = eio ? a.hidden : dy_recv;
    const void* y = eio ? dy_recv : a.hidden;
    hmc_grouped_gemm_args g = ragged_k(x, y, a.hidden_dw, a.group_list, s, eio ? s.inter : s.hidden, eio ? s.hidden : s.inter,
                                       a.weight_grad_f32 != 0, status);
    HMC_TRY(hmc_grouped_gemm(&g, stream));
  }
  if (a.gate_dw != nullptr) {
    HMC_REQUIRE(a.permute_out != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_grad: dW1 needs the saved received rows");
    const void* x = eio ? a.permute_out : a.grad_gate;
    const void* y = eio ? a.grad_gate : a.permute_out;
    hmc_grouped_gemm_args g = ragged_k(x, y, a.gate_dw, a.group_list, s, eio ? s.hidden : 2 * s.inter,
                                       eio ? 2 * s.inter : s.hidden, a.weight_grad_f32 != 0, status);
    HMC_TRY(hmc_grouped_gemm(&g, stream));
  }
  const void* returned = a.gate_dx;
  const float* returned_dot = a.row_dot;
  int64_t returned_rows = s.rows;
  if (fused_combine) {
    HMC_TRY(hmc_ep_wait(ctrl + HMC_CTRL_COMBINE, static_cast<int32_t>(s.routed * hmc_grouped_gemm_combine_units(s.hidden)),
                        t.wait_budget_ns, status, stream));
    returned = a.grad_x;
    returned_rows = t.combine_rows_limit;
  } else if (!ep1) {
    hmc_ep_combine_args c;
    memset(&c, 0, sizeof(c));
    c.results = a.gate_dx;
    c.segment_start = a.recv_segment_start;
    c.combine_target_off = a.combine_target_off;
    c.rows = s.received;
    c.hidden = s.hidden;
    c.ep = t.ep;
    c.local_experts = s.local;
    c.target_rows_limit = t.combine_rows_limit;
    c.peer_buffers = t.peer_combine;
    c.peer_ctrl = t.peer_ctrl;
    c.local_ctrl = ctrl;
    c.generation = t.generation;
    c.budget_ns = t.wait_budget_ns;
    c.status = status;
    c.result_values = a.row_dot;
    c.value_plane_offset = t.combine_plane_offset;
    HMC_TRY(hmc_ep_combine(&c, stream));
    HMC_TRY(hmc_ep_wait(ctrl + HMC_CTRL_COMBINE, static_cast<int32_t>(s.routed), t.wait_budget_ns, status, stream));
    returned = a.grad_x;
    returned_rows = t.combine_rows_limit;
    returned_dot = reinterpret_cast<const float*>(static_cast<const unsigned char*>(a.grad_x) + t.combine_plane_offset);
  }
  (void)returned_rows;
  if (a.grad_hidden != nullptr && s.tokens > 0)
    HMC_TRY(hmc_moe_token_permute_grad(returned, a.mapping, s.tokens, s.top_k, s.hidden, a.grad_hidden, status, stream));
  if (before_fc2 && a.grad_probs != nullptr && s.routed > 0) {
    // the probability gradient of route (t, k) sits at that route's row of the source order
    // (backends/bf16/autograd.py:725-730)
    HMC_REQUIRE(a.mapping != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_grad: grad_probs needs mapping");
    HMC_TRY(gather_floats(a.grad_probs, returned_dot, a.mapping, s.routed, ep1 ? s.rows : t.combine_rows_limit, status,
                          stream));
  }
  return 0;
}

// ================================================================================================ MXFP8
namespace hmc {
namespace {

struct MxExchange {
  const void* rows;   // received rows (bf16), expert-major on the owner
};

// Rows to their owners, complete before anything reads them: the MX quantiser has no per-expert gate of
// its own, so the arrival counters are awaited in a small kernel between dispatch and quantiser.
int mx_exchange(const hmc_moe_transport& t, const Shape& s, const void* src, const int32_t* src_index,
                const int32_t* expert_of_row, const int64_t* src_off, const int64_t* target_off,
                const int64_t* group_list, const int64_t* recv_segment_start, const int64_t* combine_target_off,
                void* dispatch_buffer, int32_t* ctrl, int32_t* status, cudaStream_t stream, const void** received,
                const int32_t* skip_flag = nullptr) {
  const bool ep1 = t.ep == 1;
  if (ep1) {
    if (src_index == nullptr) {
      *received = src;  // already in the owner's (= the source's) order
      return 0;
    }
    if (s.routed > 0) HMC_TRY(hmc_moe_gather_rows(src, src_index, s.routed, s.top_k, s.hidden, dispatch_buffer, stream));
    *received = dispatch_buffer;
    return 0;
  }
  HMC_TRY(begin_call(t, ctrl, stream));
  *received = dispatch_buffer;
  if (t.dispatch_mode == HMC_MOE_DISPATCH_PULL) {
    void* source = t.peer_dispatch[t.rank];
    if (s.routed > 0) {
      if (src_index != nullptr)
        HMC_TRY(hmc_moe_gather_rows(src, src_index, s.routed, s.top_k, s.hidden, source, stream));
      else if (src != source)
        HMC_CUDA_OK(cudaMemcpyAsync(source, src, static_cast<size_t>(s.routed) * s.hidden * 2, cudaMemcpyDeviceToDevice,
                                    stream));
    }
    return pull_rows(t, s, recv_segment_start, combine_target_off, dispatch_buffer, nullptr, ctrl, status, stream);
  }
  HMC_REQUIRE(t.peer_dispatch[t.rank] == dispatch_buffer, HMC_ERR_INVALID,
              "the dispatch buffer must be this rank's entry of transport.peer_dispatch");
  hmc_ep_dispatch_args d = make_dispatch(t, src, src_index, expert_of_row, src_off, target_off, s, ctrl, status, nullptr,
                                         skip_flag);
  HMC_TRY(hmc_ep_dispatch(&d, stream));
  return hmc_ep_wait_groups_unless(ctrl + HMC_CTRL_ARRIVAL, group_list, s.local, t.wait_budget_ns, status, skip_flag, stream);
}

hmc_mx_quant_args mx_quant_args(int kind, const Shape& s, int64_t pad_blocks, int64_t width, const void* src,
                                const void* aux, const int64_t* group_list, void* row_data, void* row_scale,
                                void* col_data, void* col_scale, const int32_t* skip_flag = nullptr) {
  hmc_mx_quant_args q;
  memset(&q, 0, sizeof(q));
  q.kind = kind;
  q.groups = static_cast<int32_t>(s.local);
  q.rows = s.received;
  q.pad_blocks = pad_blocks;
  q.width = width;
  q.src = src;
  q.aux = aux;
  q.group_ends = group_list;
  q.skip_flag = skip_flag;
  q.row_data = row_data;
  q.row_scale = row_scale;
  q.col_data = col_data;
  q.col_scale = col_scale;
  return q;
}

hmc_mx_gemm_args mx_gemm_args(int mode, int b_major, int epilogue, const Shape& s, int64_t pad_blocks, int64_t m,
                              int64_t n, int64_t k, const void* a, const void* a_scale, const void* b,
                              const void* b_scale, void* c, const int64_t* group_list, int32_t* status,
                              const int32_t* skip_flag = nullptr) {
  hmc_mx_gemm_args g;
  memset(&g, 0, sizeof(g));
  g.mode = mode;
  g.b_major = b_major;
  g.epilogue = epilogue;
  g.groups = static_cast<int32_t>(s.local);
  g.rows = s.received;
  g.pad_blocks = pad_blocks;
  g.m = m;
  g.n = n;
  g.k = k;
  g.a = a;
  g.a_scale = a_scale;
  g.b = b;
  g.b_scale = b_scale;
  g.c = c;
  g.group_ends = group_list;
  g.status = status;
  g.skip_flag = skip_flag;
  return g;
}

}  // namespace
}  // namespace hmc

// dispatch -> quant X -> GEMM1 -> SwiGLU + quant -> GEMM2 (+ combine) -> Top-K sum
// (reference graph: hyper_multicore/modules/mega_moe/backends/mxfp8/graph.py:140-146)
extern "C" int hmc_mega_moe_mxfp8(const hmc_mega_moe_mxfp8_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_mxfp8: null args");
  const hmc_mega_moe_mxfp8_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  Shape s;
  HMC_TRY(check_shape("hmc_mega_moe_mxfp8", a.ep, a.rank_id, a.expert_num, a.hidden_size, a.intermediate_size, a.seq_size,
                      a.top_k, a.routed_rows, a.received_rows, &s));
  HMC_REQUIRE(s.hidden % 128 == 0 && s.inter % 128 == 0, HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8: hidden and intermediate sizes must be multiples of 128");
  HMC_REQUIRE((a.source_buffer || a.routed_rows == 0) && a.w1_col_data && a.w2_col_data && a.w1_col_scale && a.w2_col_scale && a.group_list && a.up &&
                  a.a_row && a.a_scale && a.x_row && a.x_scale && a.all_event_counters,
              HMC_ERR_INVALID, "hmc_mega_moe_mxfp8: null tensor pointer");
  HMC_REQUIRE((a.x_col == nullptr) == (a.x_col_scale == nullptr) && (a.a_col == nullptr) == (a.a_col_scale == nullptr),
              HMC_ERR_INVALID, "hmc_mega_moe_mxfp8: column-quantised data and scales go together");
  const bool ep1 = a.ep == 1;
  HMC_TRY(check_transport(a.transport, "hmc_mega_moe_mxfp8", a.ep, a.rank_id, a.all_event_counters, !ep1));
  const hmc_moe_transport& t = *a.transport;
  HMC_REQUIRE(ep1 ? a.down != nullptr : (a.routed_buffer && a.recv_segment_start && a.combine_target_off &&
                                         (a.expert_of_row || s.routed == 0) && a.dispatch_buffer),
              HMC_ERR_INVALID, "hmc_mega_moe_mxfp8: missing output or combine tables");
  HMC_REQUIRE(a.pad_blocks >= (s.received + 127) / 128, HMC_ERR_INVALID, "hmc_mega_moe_mxfp8: pad_blocks too small");
  HMC_REQUIRE(a.output == nullptr || (a.mapping && a.topk_probs), HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8: the Top-K sum needs mapping and topk_probs");
  int32_t* ctrl = a.all_event_counters;
  int32_t* status = a.diagnostic_buffer;
  SideCopies copies;
  HMC_TRY(copies.init(stream, t.copy_stream));
  const void* x_recv = nullptr;
  HMC_TRY(mx_exchange(t, s, a.source_buffer, a.dispatch_src_index, a.expert_of_row, a.dispatch_src_off, a.dispatch_target_off,
                      a.group_list, a.recv_segment_start, a.combine_target_off, a.dispatch_buffer, ctrl, status, stream,
                      &x_recv, a.skip_flag));
  hmc_gemm_combine combine;
  if (s.received > 0) {
    hmc_mx_quant_args q = mx_quant_args(HMC_MXQ_PLAIN, s, a.pad_blocks, s.hidden, x_recv, nullptr, a.group_list, a.x_row,
                                        a.x_scale, a.x_col, a.x_col_scale, a.skip_flag);
    HMC_TRY(hmc_mx_quant(&q, stream));
    // GMM1 quantises bf16(silu(gate) * up) in its own epilogue (U is written once and not read again in this call);
    // HMC_MX_FUSED_SWIGLU=0 keeps the plain GEMM followed by the stand-alone SwiGLU quantiser.
    static const bool fused_swiglu = [] {
      const char* v = getenv("HMC_MX_FUSED_SWIGLU");
      return v == nullptr || v[0] != '0';
    }();
    hmc_mx_gemm_args g1 = mx_gemm_args(HMC_GEMM_RAGGED_M, HMC_MAJOR_MN, fused_swiglu ? HMC_EPI_SWIGLU_MXQ : HMC_EPI_STORE_BF16, s,
                                       a.pad_blocks, 0, 2 * s.inter, s.hidden, a.x_row, a.x_scale, a.w1_col_data,
                                       a.w1_col_scale, a.up, a.group_list, status, a.skip_flag);
    if (fused_swiglu) {
      g1.act_row_data = a.a_row;
      g1.act_row_scale = a.a_scale;
      g1.act_col_data = a.a_col;
      g1.act_col_scale = a.a_col_scale;
    }
    HMC_TRY(hmc_mx_gemm(&g1, stream));
    if (!fused_swiglu) {
      hmc_mx_quant_args qa = mx_quant_args(HMC_MXQ_SWIGLU, s, a.pad_blocks, s.inter, a.up, nullptr, a.group_list, a.a_row,
                                           a.a_scale, a.a_col, a.a_col_scale, a.skip_flag);
      HMC_TRY(hmc_mx_quant(&qa, stream));
    }
    hmc_mx_gemm_args g2 = mx_gemm_args(HMC_GEMM_RAGGED_M, HMC_MAJOR_MN, HMC_EPI_STORE_BF16, s, a.pad_blocks, 0, s.hidden,
                                       s.inter, a.a_row, a.a_scale, a.w2_col_data, a.w2_col_scale, ep1 ? a.down : nullptr,
                                       a.group_list, status, a.skip_flag);
    if (!ep1) {
      combine = make_combine(t, a.recv_segment_start, a.combine_target_off, s.local);
      g2.combine = &combine;
    }
    HMC_TRY(hmc_mx_gemm(&g2, stream));
  }
  const void* routed = a.down;
  if (!ep1) {
    HMC_TRY(hmc_ep_wait_unless(ctrl + HMC_CTRL_COMBINE, static_cast<int32_t>(s.routed * hmc_mx_gemm_combine_units(s.hidden)),
                               t.wait_budget_ns, status, a.skip_flag, stream));
    routed = a.routed_buffer;
    if (a.saved_combine != nullptr) {
      HMC_TRY(copies.begin());
      // (a call that does not fit the workspace is a no-op on the device: copy no more than the buffer holds)
      const int64_t held = s.routed < t.combine_rows_limit ? s.routed : t.combine_rows_limit;
      HMC_TRY(copies.copy(a.saved_combine, a.routed_buffer, static_cast<size_t>(held) * s.hidden * 2));
    }
  }
  if (a.output != nullptr && s.tokens > 0)
    HMC_TRY(moe_unpermute_unless(routed, a.mapping, a.topk_probs, s.tokens, s.top_k, s.hidden,
                                 ep1 ? s.rows : t.combine_rows_limit, a.output, status, a.skip_flag, stream));
  return copies.end();
}

// dY rows + dProbs -> dispatch -> quant -> dA -> SwiGLU-grad + quant -> dX (+ combine), dW2, dW1 -> Top-K sum
// (reference graph: backends/mxfp8/graph.py:147-154)
extern "C" int hmc_mega_moe_mxfp8_grad(const hmc_mega_moe_mxfp8_grad_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mega_moe_mxfp8_grad: null args");
  const hmc_mega_moe_mxfp8_grad_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  Shape s;
  HMC_TRY(check_shape("hmc_mega_moe_mxfp8_grad", a.ep, a.rank_id, a.expert_num, a.hidden_size, a.intermediate_size,
                      a.seq_size, a.top_k, a.routed_rows, a.received_rows, &s));
  HMC_REQUIRE(s.hidden % 128 == 0 && s.inter % 128 == 0, HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8_grad: hidden and intermediate sizes must be multiples of 128");
  HMC_REQUIRE(a.source && a.w2_row_data && a.w2_row_scale && a.w1_row_data && a.w1_row_scale && a.da && a.up && a.group_list &&
                  a.dy_row && a.dy_scale && a.du_row && a.du_scale && a.all_event_counters,
              HMC_ERR_INVALID, "hmc_mega_moe_mxfp8_grad: null tensor pointer");
  const bool want_dw = a.dw1 != nullptr || a.dw2 != nullptr;
  HMC_REQUIRE(!want_dw || (a.dy_col && a.dy_col_scale && a.du_col && a.du_col_scale), HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8_grad: weight gradients need the column-quantised dY and dU buffers");
  HMC_REQUIRE(a.dw2 == nullptr || s.received == 0 || (a.a_col && a.a_col_scale), HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8_grad: dW2 needs the column-quantised activation saved by forward");
  HMC_REQUIRE(a.dw1 == nullptr || s.received == 0 || (a.x_col && a.x_col_scale), HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8_grad: dW1 needs the column-quantised input saved by forward");
  const bool ep1 = a.ep == 1;
  HMC_TRY(check_transport(a.transport, "hmc_mega_moe_mxfp8_grad", a.ep, a.rank_id, a.all_event_counters, !ep1));
  const hmc_moe_transport& t = *a.transport;
  HMC_REQUIRE(ep1 ? a.dx != nullptr : (a.routed_buffer && a.recv_segment_start && a.combine_target_off &&
                                       (a.expert_of_row || s.routed == 0) && a.dispatch),
              HMC_ERR_INVALID, "hmc_mega_moe_mxfp8_grad: missing output or combine tables");
  HMC_REQUIRE(a.grad_output == nullptr || (a.mapping && a.topk_probs && a.grad_probs && a.saved_combine), HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8_grad: the prologue needs mapping, topk_probs, grad_probs and saved_combine");
  HMC_REQUIRE(a.grad_hidden == nullptr || a.mapping != nullptr, HMC_ERR_INVALID,
              "hmc_mega_moe_mxfp8_grad: the Top-K sum of dX needs mapping");
  int32_t* ctrl = a.all_event_counters;
  int32_t* status = a.diagnostic_buffer;
  if (a.grad_output != nullptr && s.tokens > 0)
    HMC_TRY(hmc_moe_unpermute_grad(a.saved_combine, a.grad_output, a.mapping, a.topk_probs, s.tokens, s.top_k, s.hidden,
                                   a.source, a.grad_probs, status, stream));
  const void* dy_recv = nullptr;
  HMC_TRY(mx_exchange(t, s, a.source, nullptr, a.expert_of_row, a.dispatch_src_off, a.dispatch_target_off, a.group_list,
                      a.recv_segment_start, a.combine_target_off, a.dispatch, ctrl, status, stream, &dy_recv));
  const int wepi = a.weight_grad_f32 ? HMC_EPI_STORE_F32 : HMC_EPI_STORE_BF16;
  hmc_gemm_combine combine;
  if (s.received > 0) {
    hmc_mx_quant_args q = mx_quant_args(HMC_MXQ_PLAIN, s, a.pad_blocks, s.hidden, dy_recv, nullptr, a.group_list, a.dy_row,
                                        a.dy_scale, want_dw ? a.dy_col : nullptr, want_dw ? a.dy_col_scale : nullptr);
    HMC_TRY(hmc_mx_quant(&q, stream));
    // W2 [e, I, H] row-quantised (blocks along H) is the K-major B of dA = dY . W2^T. The GEMM can also produce
    // the quantised dU = SwiGLU-grad(dA, U) in its epilogue (HMC_MX_FUSED_SWIGLU_GRAD=1, I a multiple of 256), but
    // eight epilogue warps per SM evaluate the sigmoids and the two quantisations more slowly than the stand-alone
    // quantiser's full grid does (dA 390 us against 134 + 87 us on the 4096-token bench shape): off by default.
    static const bool fused_allowed = [] {
      const char* v = getenv("HMC_MX_FUSED_SWIGLU_GRAD");
      return v != nullptr && v[0] == '1';
    }();
    const bool fused_grad = fused_allowed && s.inter % 256 == 0;
    hmc_mx_gemm_args g1 = mx_gemm_args(HMC_GEMM_RAGGED_M, HMC_MAJOR_K, fused_grad ? HMC_EPI_SWIGLU_GRAD_MXQ : HMC_EPI_STORE_BF16,
                                       s, a.pad_blocks, 0, s.inter, s.hidden, a.dy_row, a.dy_scale, a.w2_row_data,
                                       a.w2_row_scale, fused_grad ? nullptr : a.da, a.group_list, status);
    if (fused_grad) {
      g1.aux = a.up;
      g1.act_row_data = a.du_row;
      g1.act_row_scale = a.du_scale;
      g1.act_col_data = want_dw ? a.du_col : nullptr;
      g1.act_col_scale = want_dw ? a.du_col_scale : nullptr;
    }
    HMC_TRY(hmc_mx_gemm(&g1, stream));
    if (!fused_grad) {
      hmc_mx_quant_args qu = mx_quant_args(HMC_MXQ_SWIGLU_GRAD, s, a.pad_blocks, 2 * s.inter, a.da, a.up, a.group_list,
                                           a.du_row, a.du_scale, want_dw ? a.du_col : nullptr,
                                           want_dw ? a.du_col_scale : nullptr);
      HMC_TRY(hmc_mx_quant(&qu, stream));
    }
    hmc_mx_gemm_args g2 = mx_gemm_args(HMC_GEMM_RAGGED_M, HMC_MAJOR_K, HMC_EPI_STORE_BF16, s, a.pad_blocks, 0, s.hidden,
                                       2 * s.inter, a.du_row, a.du_scale, a.w1_row_data, a.w1_row_scale,
                                       ep1 ? a.dx : nullptr, a.group_list, status);
    if (!ep1) {
      combine = make_combine(t, a.recv_segment_start, a.combine_target_off, s.local);
      g2.combine = &combine;
    }
    HMC_TRY(hmc_mx_gemm(&g2, stream));
    if (a.dw2 != nullptr) {
      hmc_mx_gemm_args gw = mx_gemm_args(HMC_GEMM_RAGGED_K, HMC_MAJOR_MN, wepi, s, a.pad_blocks, s.inter, s.hidden, 0,
                                         a.a_col, a.a_col_scale, a.dy_col, a.dy_col_scale, a.dw2, a.group_list, status);
      HMC_TRY(hmc_mx_gemm(&gw, stream));
    }
    if (a.dw1 != nullptr) {
      hmc_mx_gemm_args gw = mx_gemm_args(HMC_GEMM_RAGGED_K, HMC_MAJOR_MN, wepi, s, a.pad_blocks, s.hidden, 2 * s.inter, 0,
                                         a.x_col, a.x_col_scale, a.du_col, a.du_col_scale, a.dw1, a.group_list, status);
      HMC_TRY(hmc_mx_gemm(&gw, stream));
    }
  } else {
    const size_t element = a.weight_grad_f32 ? 4 : 2;
    if (a.dw1 != nullptr)
      HMC_CUDA_OK(cudaMemsetAsync(a.dw1, 0, static_cast<size_t>(s.local) * s.hidden * 2 * s.inter * element, stream));
    if (a.dw2 != nullptr)
      HMC_CUDA_OK(cudaMemsetAsync(a.dw2, 0, static_cast<size_t>(s.local) * s.inter * s.hidden * element, stream));
  }
  const void* returned = a.dx;
  if (!ep1) {
    HMC_TRY(hmc_ep_wait(ctrl + HMC_CTRL_COMBINE, static_cast<int32_t>(s.routed * hmc_mx_gemm_combine_units(s.hidden)),
                        t.wait_budget_ns, status, stream));
    returned = a.routed_buffer;
  }
  if (a.grad_hidden != nullptr && s.tokens > 0)
    HMC_TRY(hmc_moe_token_permute_grad(returned, a.mapping, s.tokens, s.top_k, s.hidden, a.grad_hidden, status, stream));
  return 0;
}
