"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE.

Usage (needs the reference tree; it is imported, never copied):

    PYTHONPATH=/path/to/xkernels/src python tests/golden/make_golden.py

Every case stores the exact inputs and the outputs of the reference's own
callables (``xkernels.ops.moe`` reference backend) on CPU, with inputs from the
reference's seeded harness generators (``registry/input_gen.py``, seed 1729 as
in ``verify.py:26``) where one exists.  The fixtures pin ``oracle/moe_oracle.py``
and are compared against the CUDA kernels by the GPU tests.
"""

from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from tests.golden.golden_io import GOLDEN_DIR, save_case  # noqa: E402

import xkernels  # noqa: E402,F401  (the reference)
from xkernels.ops.moe.mxfp4 import make_mxfp4_moe_weights  # noqa: E402
from xkernels.ops.moe.mxfp4_reference import moe_mxfp4_ref  # noqa: E402
from xkernels.ops.moe.reference import moe_w4a16_ref  # noqa: E402
from xkernels.ops.moe.sum_reduce import moe_sum_reduce_ref  # noqa: E402
from xkernels.ops.moe.topk_softmax import topk_softmax_ref  # noqa: E402
from xkernels.ops.moe.w4a16 import (  # noqa: E402
    dequant_w4a16,
    moe_align_block_size_ep,
    moe_align_block_size_ref,
)
from xkernels.registry.input_gen import generate_inputs  # noqa: E402
from xkernels.registry.loader import load_shape_sweep  # noqa: E402

from xkernels_b200 import synth  # noqa: E402

SEED = 1729
manifest = {}


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def sweep_points(name):
    return [dict(p) for p in load_shape_sweep(name)]


# ---- moe_align_block_size ---------------------------------------------------
def gen_align():
    for i, pt in enumerate(sweep_points("moe_align_block_size")):
        inp = generate_inputs("moe_align_block_size@1.0.0", pt, SEED, "cpu")
        s, e, n = moe_align_block_size_ref(**inp)
        if inp["topk_ids"].numel() > 20000:
            # large point: keep the seed-regenerable input's digest and the output digest only
            manifest[f"align_sweep{i}"] = {
                "point": pt, "input_sha256": digest(inp["topk_ids"]), "output_sha256": digest(s, e, n)}
            continue
        save_case(f"align_sweep{i}", {**inp, "sorted_ids": s, "expert_ids": e, "num_post": n})
    # hand-checkable known answer
    ids = torch.tensor([[1, 0], [1, 1]], dtype=torch.int32)
    s, e, n = moe_align_block_size_ref(ids, 2, 2)
    save_case("align_kat", {"topk_ids": ids, "block_size": 2, "num_experts": 2, "truncate": True,
                            "sorted_ids": s, "expert_ids": e, "num_post": n})
    # skewed routing with empty experts, both truncate modes
    g = torch.Generator().manual_seed(SEED)
    ids = torch.randint(0, 5, (300, 4), generator=g, dtype=torch.int32) * 3  # experts 0,3,6,9,12 of 16
    for trunc in (True, False):
        s, e, n = moe_align_block_size_ref(ids, 16, 16, truncate=trunc)
        save_case(f"align_skew_trunc{int(trunc)}", {"topk_ids": ids, "block_size": 16, "num_experts": 16,
                                                     "truncate": trunc, "sorted_ids": s, "expert_ids": e,
                                                     "num_post": n})
    # expert-parallel form: 2 ranks over 8 experts
    ids = torch.randint(0, 8, (37, 3), generator=g, dtype=torch.int32)
    for rank in range(2):
        emap = torch.full((8,), -1, dtype=torch.int32)
        emap[rank * 4:(rank + 1) * 4] = torch.arange(4, dtype=torch.int32)
        s, e, n = moe_align_block_size_ep(ids, 16, 8, emap)
        save_case(f"align_ep_rank{rank}", {"topk_ids": ids, "block_size": 16, "num_experts": 8,
                                           "expert_map": emap, "sorted_ids": s, "expert_ids": e,
                                           "num_post": n})
    # a rank that owns no expert
    emap = torch.full((8,), -1, dtype=torch.int32)
    s, e, n = moe_align_block_size_ep(ids, 16, 8, emap)
    save_case("align_ep_empty", {"topk_ids": ids, "block_size": 16, "num_experts": 8, "expert_map": emap,
                                 "sorted_ids": s, "expert_ids": e, "num_post": n})


# ---- moe_int4_w4a16 ----------------------------------------------------------
def gen_int4():
    for i, pt in enumerate(sweep_points("moe_int4_w4a16")):
        inp = generate_inputs("moe_int4_w4a16@1.0.0", pt, SEED, "cpu")
        out = moe_w4a16_ref(**inp)
        save_case(f"int4_sweep{i}", {**inp, "out": out})
    # dequant known answers: words 0x76543210 / 0xFEDCBA98 with scale 0.5 and 2
    packed = torch.tensor([[[0x76543210, 0xFEDCBA98 - (1 << 32)] * 4]], dtype=torch.int32)  # [1,1,8] -> K=64
    scale = torch.tensor([[[0.5, 2.0]]], dtype=torch.bfloat16)
    save_case("int4_dequant_kat", {"packed": packed, "scale": scale, "group_size": 32,
                                   "w_bf16": dequant_w4a16(packed, scale, 32),
                                   "w_fp32": dequant_w4a16(packed, scale, 32, out_dtype=torch.float32)})
    # tiny benchmark configuration (M=16,K=512,N=256,E=8,top_k=2), distinct top-k ids
    inp = synth.make_int4(synth.CONFIGS["int4_tiny"], seed=SEED)
    out = moe_w4a16_ref(**inp)
    save_case("int4_tiny", {**inp, "out": out})
    out_nw = moe_w4a16_ref(**inp, mul_routed_weight=False)
    save_case("int4_tiny_noweight", {"out": out_nw})
    # replicated expert-parallel partials: 2 ranks x 4 experts
    for rank in range(2):
        emap = torch.full((8,), -1, dtype=torch.int32)
        emap[rank * 4:(rank + 1) * 4] = torch.arange(4, dtype=torch.int32)
        sl = slice(rank * 4, (rank + 1) * 4)
        part = moe_w4a16_ref(inp["A"], inp["packed"][sl], inp["scale"][sl], inp["topk_ids"], inp["topk_w"],
                             group_size=32, expert_map=emap)
        save_case(f"int4_tiny_ep_rank{rank}", {"expert_map": emap, "out": part})


# ---- moe_mxfp4 -----------------------------------------------------------------
def gen_mxfp4():
    g = torch.Generator().manual_seed(SEED)
    for name, (E, hidden, ispp, M, top_k, bias, dt) in {
        "mxfp4_small": (4, 64, 32, 5, 2, False, torch.bfloat16),
        "mxfp4_small_bias": (4, 64, 32, 5, 2, True, torch.bfloat16),
        "mxfp4_mid": (8, 256, 256, 24, 3, True, torch.bfloat16),
        "mxfp4_fp32_act": (4, 96, 64, 7, 2, False, torch.float32),
    }.items():
        wts = make_mxfp4_moe_weights(E, hidden, ispp, with_bias=bias, device="cpu", seed=SEED + 1)
        A = torch.randn(M, hidden, generator=g).to(dt)
        ids = torch.stack([torch.randperm(E, generator=g)[:top_k] for _ in range(M)]).to(torch.int32)
        w = torch.rand(M, top_k, generator=g, dtype=torch.float32)
        kw = dict(A=A, w13=wts["w13"], w13_scale=wts["w13_scale"], w2=wts["w2"], w2_scale=wts["w2_scale"],
                  topk_ids=ids, topk_w=w, b13=wts["b13"], b2=wts["b2"], swiglu_limit=10.0)
        out = moe_mxfp4_ref(**kw)
        save_case(name, {**kw, "out": out})
    # wide scale range incl. the 0xFF (-> 0) code, byte 0 and large exponents; limit disabled
    cfg = synth.Mxfp4Config("x", M=9, hidden=128, ispp=64, E=6, top_k=3, scale_lo=120, scale_hi=131)
    kw = synth.make_mxfp4(cfg, seed=SEED)
    kw["w13_scale"][0, 0, 0] = 0xFF
    kw["w2_scale"][1, 3, 1] = 0xFF
    kw["w13_scale"][2, 5, 2] = 0
    out = moe_mxfp4_ref(**kw, swiglu_limit=None)
    save_case("mxfp4_scales", {**kw, "swiglu_limit": 0.0, "out": out})


def gen_mxfp4_tensor_core_shape():
    """A case whose dimensions are multiples of 512 (what the tcgen05 path of this repo takes: a row's
    e8m0 scales must be whole 16-byte TMA rows), with bias, the clamp, and the edge scale codes."""
    cfg = synth.Mxfp4Config("x", M=20, hidden=512, ispp=512, E=4, top_k=2, scale_lo=118, scale_hi=131)
    kw = synth.make_mxfp4(cfg, seed=SEED + 40, with_bias=True)
    kw["w13_scale"][0, 0, 0] = 0xFF
    kw["w13_scale"][1, 700, 9] = 0xFF
    kw["w2_scale"][1, 3, 1] = 0xFF
    kw["w13_scale"][2, 5, 2] = 0
    kw["w2_scale"][3, 130, 15] = 0
    out = moe_mxfp4_ref(**kw, swiglu_limit=10.0)
    save_case("mxfp4_tc_scales", {**kw, "swiglu_limit": 10.0, "out": out})


def gen_int4_ffn():
    """The reference's own ops composed into a two-GEMM expert layer (what oracle.moe_int4_ffn restates):
    moe_w4a16_ref over the slots, SwiGLU, moe_w4a16_ref with the routing weights, moe_sum_reduce_ref."""
    import torch.nn.functional as F

    for name, (M, hidden, inter, E, top_k, dt, limit) in {
        "int4_ffn_small": (6, 64, 32, 4, 2, torch.bfloat16, None),
        "int4_ffn_tc": (24, 256, 256, 4, 3, torch.bfloat16, 7.0),
        "int4_ffn_fp32": (5, 64, 64, 3, 2, torch.float32, None),
    }.items():
        g = torch.Generator().manual_seed(SEED + M)
        A = torch.randn(M, hidden, generator=g).to(dt)
        w13, s13 = synth.int4_weights(E, 2 * inter, hidden, 32, seed=SEED + 50)
        w2, s2 = synth.int4_weights(E, hidden, inter, 32, seed=SEED + 60)
        ids = torch.stack([torch.randperm(E, generator=g)[:top_k] for _ in range(M)]).to(torch.int32)
        w = torch.rand(M, top_k, generator=g, dtype=torch.float32)
        slot_ids = ids.reshape(-1, 1)
        rows1 = moe_w4a16_ref(A.repeat_interleave(top_k, dim=0), w13, s13, slot_ids, torch.ones(M * top_k, 1),
                              group_size=32, mul_routed_weight=False)
        gate, up = rows1.float().chunk(2, dim=-1)
        if limit is not None:
            gate = torch.clamp(gate, max=limit)
            up = torch.clamp(up, min=-limit, max=limit)
        act = (F.silu(gate) * up).to(dt)
        rows2 = moe_w4a16_ref(act, w2, s2, slot_ids, w.reshape(-1, 1), group_size=32, mul_routed_weight=True)
        out = moe_sum_reduce_ref(rows2.view(M, top_k, hidden))
        save_case(name, {"A": A, "w13_packed": w13, "w13_scale": s13, "w2_packed": w2, "w2_scale": s2, "topk_ids": ids,
                         "topk_w": w, "swiglu_limit": 0.0 if limit is None else limit, "out": out})


# ---- moe_sum_reduce ---------------------------------------------------------------
def gen_sum_reduce():
    for i, pt in enumerate(sweep_points("moe_sum_reduce")):
        if pt["M"] * pt["H"] > 200000:
            continue
        inp = generate_inputs("moe_sum_reduce@1.0.0", pt, SEED, "cpu")
        save_case(f"sum_reduce_sweep{i}", {**inp, "out": moe_sum_reduce_ref(**inp)})
    g = torch.Generator().manual_seed(SEED)
    y = torch.randn(5, 3, 40, generator=g).to(torch.bfloat16)
    save_case("sum_reduce_noweight", {"y": y, "w": None, "routed_scaling_factor": 2.5,
                                      "out": moe_sum_reduce_ref(y, None, 2.5)})
    w = torch.randn(5, 3, generator=g).to(torch.bfloat16)
    save_case("sum_reduce_bf16w", {"y": y, "w": w, "routed_scaling_factor": 1.0,
                                   "out": moe_sum_reduce_ref(y, w, 1.0)})


# ---- topk_softmax (router) ---------------------------------------------------------
def gen_topk_softmax():
    def store(name, gating, topk, renorm):
        w, ids = topk_softmax_ref(gating, topk, renorm)
        save_case(name, {"gating_output": gating, "topk": topk, "renormalize": renorm, "topk_weights": w,
                         "topk_ids": ids})

    for i, pt in enumerate(sweep_points("topk_softmax")):
        inp = generate_inputs("topk_softmax@1.0.0", pt, SEED, "cpu")
        store(f"topk_softmax_sweep{i}", inp["gating_output"], inp["topk"], inp["renormalize"])
    g = torch.Generator().manual_seed(SEED)
    # heavy ties: logits on a 0.5 grid, so many experts share a probability exactly
    coarse = (torch.randn(64, 256, generator=g) * 2).round() / 2
    store("topk_softmax_ties_bf16", coarse.to(torch.bfloat16), 8, True)
    store("topk_softmax_ties_fp16", coarse[:, :48].to(torch.float16), 5, False)
    # every expert equal: the first topk ids win
    store("topk_softmax_all_equal", torch.full((3, 40), 0.25), 6, True)
    # non power-of-two expert count, more than 32 selected, both renormalisation modes
    wide = torch.randn(9, 1000, generator=g)
    store("topk_softmax_wide_renorm", wide, 40, True)
    store("topk_softmax_wide_raw", wide, 40, False)
    # one expert, one token
    store("topk_softmax_single", torch.randn(1, 1, generator=g), 1, True)


if __name__ == "__main__":
    torch.manual_seed(0)
    if "--only-topk-softmax" in sys.argv:      # add the router fixtures without touching the others
        gen_topk_softmax()
        print("wrote the topk_softmax cases")
        sys.exit(0)
    if "--only-int4-ffn" in sys.argv:          # add the two-GEMM INT4 cases without touching the others
        gen_int4_ffn()
        print("wrote the int4_ffn cases")
        sys.exit(0)
    if "--only-mxfp4-tc" in sys.argv:          # add the 512-multiple MXFP4 case without touching the others
        gen_mxfp4_tensor_core_shape()
        print("wrote mxfp4_tc_scales")
        sys.exit(0)
    gen_align()
    gen_int4()
    gen_mxfp4()
    gen_mxfp4_tensor_core_shape()
    gen_int4_ffn()
    gen_sum_reduce()
    gen_topk_softmax()
    (GOLDEN_DIR / "manifest.json").write_text(json.dumps(manifest, indent=1, sort_keys=True))
    total = sum(p.stat().st_size for p in GOLDEN_DIR.glob("*.npz"))
    print(f"wrote {len(list(GOLDEN_DIR.glob('*.npz')))} cases, {total / 1e6:.2f} MB")
