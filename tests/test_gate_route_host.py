"""CPU: the Route that runs inside the gate projection's epilogue, compiled for the host.

The marked region of csrc/gate_promoted.cu (the launch parameters, route_token and route_pair) is plain C++ apart
from a few intrinsics. This test compiles it with g++ and stand-ins for those - two host threads play the lanes
l and l + 16 of route_pair, a shuffle is an exchange through two slots - and checks both variants against the
fixtures generated from the reference's MegaGate (tests/golden/gate.npz) and against the oracle on seeded inputs:
expert sets exact wherever the top-k margin is clear, weights within rtol 1e-5 / atol 1e-6, and the two variants
equal to each other bit for bit.
"""

from __future__ import annotations

import ctypes
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import gate as ogate
from tests.helpers import load_cases, sorted_sets

ROOT = Path(__file__).resolve().parents[1]
SOURCE = ROOT / "hyper_multicore_b200" / "csrc" / "gate_promoted.cu"
SCORING = {"sqrtsoftplus": 0, "softmax": 1, "sigmoid": 2}

PRELUDE = r"""
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <barrier>
#include <thread>
#include "hmc_b200.h"
#define __device__
#define __forceinline__ inline
#define __ldg(p) (*(p))
#define __fadd_rn(a, b) ((a) + (b))
static inline int __float_as_int(float f) { int i; memcpy(&i, &f, 4); return i; }
struct float4 { float x, y, z, w; };
static inline float4 make_float4(float a, float b, float c, float d) { float4 r = {a, b, c, d}; return r; }
constexpr int GN = 64, GM = 128, G_STAGES = 4, G_STAGE_BYTES = 40960;
static std::barrier<> g_bar(2);
static uint32_t g_slot[2];
static thread_local int g_half;
template <class T> static T exchange_with_partner(T x) {
  uint32_t w; memcpy(&w, &x, 4);
  g_slot[g_half] = w; g_bar.arrive_and_wait();
  const uint32_t o = g_slot[g_half ^ 1]; g_bar.arrive_and_wait();
  T r; memcpy(&r, &o, 4); return r;
}
#define __shfl_xor_sync(mask, x, offset) exchange_with_partner(x)
"""

DRIVER = r"""
extern "C" int params_size() { return (int)sizeof(GateParams); }
extern "C" void route_one_thread(const float* logits, GateParams* p) {
  for (long long t = 0; t < p->tokens; ++t) {
    float v[GN];
    for (int c = 0; c < GN; ++c) v[c] = c < p->experts ? logits[t * p->experts + c] : 0.f;
    route_token(v, t, *p);
  }
}
extern "C" void route_two_threads(const float* logits, GateParams* p) {
  auto lane = [&](int half) {
    g_half = half;
    for (long long t = 0; t < p->tokens + 3; ++t) {  // three rows past the end: math runs, nothing is stored
      float v[32];
      for (int i = 0; i < 32; ++i) {
        const int c = 32 * half + i;
        v[i] = (t < p->tokens && c < p->experts) ? logits[t * p->experts + c] : 0.f;
      }
      route_pair(v, half, t, t < p->tokens, *p);
    }
  };
  std::thread a(lane, 0), b(lane, 1);
  a.join();
  b.join();
}
"""


class _Params(ctypes.Structure):
    _fields_ = [("tokens", ctypes.c_longlong), ("hidden", ctypes.c_int), ("experts", ctypes.c_int),
                ("epad", ctypes.c_int), ("parts", ctypes.c_int), ("k_blocks", ctypes.c_int),
                ("k_per_slice", ctypes.c_int), ("logits", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("text_bias", ctypes.c_void_p), ("vision_bias", ctypes.c_void_p), ("image_mask", ctypes.c_void_p),
                ("use_vision_bias", ctypes.c_int), ("top_k", ctypes.c_int), ("scoring", ctypes.c_int),
                ("scale", ctypes.c_float), ("weights", ctypes.c_void_p), ("indices", ctypes.c_void_p),
                ("route_scores", ctypes.c_void_p), ("selected", ctypes.c_void_p), ("denominator", ctypes.c_void_p)]


@pytest.fixture(scope="module")
def host_route(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    text = SOURCE.read_text()
    begin = text.index("// [host-testable begin]")
    end = text.index("// [host-testable end]")
    build = tmp_path_factory.mktemp("gate_route_host")
    source = build / "gate_route_host.cpp"
    source.write_text(PRELUDE + text[begin:end] + DRIVER)
    library = build / "libgate_route_host.so"
    subprocess.run(["g++", "-O2", "-std=c++20", "-pthread", "-ffp-contract=off", "-shared", "-fPIC",
                    f"-I{ROOT / 'include'}", "-o", str(library), str(source)], check=True)
    lib = ctypes.CDLL(str(library))
    assert lib.params_size() == ctypes.sizeof(_Params), "the mirror of GateParams is out of date"
    return lib


def _run(fn, logits, bias, bias_vl, mask, top_k, scoring, scale):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    tokens, experts = logits.shape
    out = {"weights": np.zeros((tokens, top_k), np.float32), "indices": np.zeros((tokens, top_k), np.int64),
           "route_scores": np.zeros((tokens, experts), np.float32), "selected": np.zeros((tokens, top_k), np.float32),
           "denominator": np.zeros((tokens, 1), np.float32), "logits": np.zeros((tokens, experts), np.float32)}
    keep = [np.ascontiguousarray(bias, dtype=np.float32),
            np.ascontiguousarray(bias if bias_vl is None else bias_vl, dtype=np.float32),
            None if mask is None else np.ascontiguousarray(mask, dtype=np.uint8)]
    p = _Params()
    p.tokens, p.experts, p.top_k, p.scoring, p.scale = tokens, experts, top_k, SCORING[scoring], scale
    p.text_bias, p.vision_bias = keep[0].ctypes.data, keep[1].ctypes.data
    p.use_vision_bias = int(mask is not None)
    p.image_mask = None if mask is None else keep[2].ctypes.data
    for name, array in out.items():
        setattr(p, name, array.ctypes.data)
    fn(logits.ctypes.data_as(ctypes.c_void_p), ctypes.byref(p))
    return out


def _both(lib, *args):
    one = _run(lib.route_one_thread, *args)
    two = _run(lib.route_two_threads, *args)
    for name in ("weights", "indices", "route_scores", "selected", "denominator"):
        assert np.array_equal(one[name], two[name], equal_nan=True), f"{name}: one and two threads per token differ"
    assert np.array_equal(two["logits"].view(np.int32), np.asarray(args[0], dtype=np.float32).view(np.int32))
    return one


def test_host_compiled_route_matches_the_reference_fixtures(host_route):
    checked = 0
    for case in load_cases("gate"):
        tokens, _, experts, top_k, vision = (int(v) for v in case["config"])
        if experts > 64:
            continue
        scale = float(case["scale"][0])
        got = _both(host_route, case["logits"].numpy(), case["bias"].numpy(),
                    case["bias_vl"].numpy() if vision else None,
                    case["mask"].numpy().reshape(-1) if vision else None, top_k, case["scoring"], scale)
        got_idx, got_w = sorted_sets(torch.from_numpy(got["indices"]), torch.from_numpy(got["weights"]))
        ref_idx, ref_w = sorted_sets(case["indices"], case["weights"])
        assert torch.equal(got_idx, ref_idx)
        torch.testing.assert_close(got_w, ref_w, rtol=1e-5, atol=1e-6)
        checked += 1
    assert checked > 0


@pytest.mark.parametrize("scoring", ["sqrtsoftplus", "softmax", "sigmoid"])
@pytest.mark.parametrize("experts,top_k", [(64, 6), (48, 48), (33, 5), (20, 1), (1, 1)])
def test_host_compiled_route_matches_the_oracle(host_route, scoring, experts, top_k):
    torch.manual_seed(experts * 7 + top_k)
    tokens = 257
    logits = torch.randn(tokens, experts)
    bias = torch.empty(experts).uniform_(-0.1, 0.1)
    bias_vl = torch.empty(experts).uniform_(-0.1, 0.1)
    mask = torch.rand(tokens) < 0.4
    ref = ogate.route_from_logits(logits, bias, bias_vl, mask, top_k, scoring, 2.5)
    got = _both(host_route, logits.numpy(), bias.numpy(), bias_vl.numpy(), mask.numpy(), top_k, scoring, 2.5)
    torch.testing.assert_close(torch.from_numpy(got["route_scores"]), ref["scores"], rtol=1e-5, atol=1e-6)
    safe = ogate.topk_margin(ref["biased"], top_k) > 1e-6
    got_idx, got_w = sorted_sets(torch.from_numpy(got["indices"]), torch.from_numpy(got["weights"]))
    ref_idx, ref_w = sorted_sets(ref["indices"], ref["weights"])
    assert torch.equal(got_idx[safe], ref_idx[safe])
    torch.testing.assert_close(got_w[safe], ref_w[safe], rtol=1e-5, atol=1e-6)


def test_host_compiled_route_ties_and_special_values(host_route):
    """Exact ties go to the lower expert; NaN orders as +inf; -inf biases never win while a finite score is left."""
    logits = np.zeros((4, 40), np.float32)
    logits[1, [7, 3, 38]] = 1.0
    logits[2, 5] = np.nan
    logits[3, :] = np.linspace(-1, 1, 40, dtype=np.float32)
    bias = np.zeros(40, np.float32)
    got = _both(host_route, logits, bias, None, None, 3, "sigmoid", 1.0)
    assert got["indices"][0].tolist() == [0, 1, 2]
    assert got["indices"][1].tolist() == [3, 7, 38]
    assert got["indices"][2][0] == 5
    bias[39] = -np.inf
    got = _both(host_route, logits, bias, None, None, 3, "sigmoid", 1.0)
    assert got["indices"][3].tolist() == [38, 37, 36]
