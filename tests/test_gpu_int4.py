"""fused_moe_int4_w4a16 on the GPU, through the C-ABI, vs the oracle and the fixtures made by
the reference.  Tolerance (written here, from the task statement and the op spec
registry/ops/moe_int4_w4a16.spec.json:30-41): bf16 outputs |a-e| <= 1e-2 + 2e-2|e| against the
fp32-accumulated reference; fp32 activations rtol = atol = 1e-3."""

import pytest
import torch

import xkernels_b200 as xkb
from oracle import moe_oracle as oracle
from tests.golden.golden_io import load_case
from tests.gpu_util import assert_within, to_dev
from xkernels_b200 import synth

pytestmark = pytest.mark.gpu
TOL = {torch.bfloat16: (2e-2, 1e-2), torch.float32: (1e-3, 1e-3)}
KEYS = ("A", "packed", "scale", "topk_ids", "topk_w")


def call(c, dev, **kw):
    d = to_dev({k: c[k] for k in KEYS}, dev)
    return xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"],
                                    group_size=int(c.get("group_size", 32)), **kw)


@pytest.mark.parametrize("name", ["int4_sweep0", "int4_sweep1", "int4_sweep2", "int4_sweep3", "int4_tiny"])
@pytest.mark.parametrize("path", ["auto", "simt"])
def test_golden(name, path, cuda_device):
    c = load_case(name)
    out = call(c, cuda_device, path=path)
    assert_within(out, c["out"], *TOL[c["A"].dtype], what=f"{name}/{path}")


@pytest.mark.parametrize("M,K,N,E,top_k,tile", [
    (16, 512, 256, 8, 2, 16),      # the tiny configuration: 4 slots per expert -> 16-token tile
    (64, 256, 128, 4, 2, 64),      # 32 slots per expert on average -> 64-token tile
    (40, 768, 384, 8, 4, 32),      # 20 per expert -> 32-token tile
    (96, 1024, 256, 6, 4, 128),    # 64 per expert -> 128-token tile, two row tiles per token tile
    (300, 512, 128, 3, 2, 128),    # 200 per expert -> 128-token tile, one row tile (N = 128)
    (7, 7168, 256, 48, 8, 16),     # decode-like K, mostly empty experts
])
def test_tensor_core_path_against_oracle(M, K, N, E, top_k, tile, cuda_device):
    """The tcgen05 kernel at every token-tile size it is instantiated for."""
    from xkernels_b200 import ops

    g = torch.Generator().manual_seed(M + K + N)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16)
    packed, scale = synth.int4_weights(E, N, K, 32, seed=M, device="cpu")
    ids, w = synth.routing(M, E, top_k, seed=K, device="cpu")
    want = oracle.moe_w4a16(A, packed, scale, ids, w, 32)
    c = {"A": A, "packed": packed, "scale": scale, "topk_ids": ids, "topk_w": w}
    got = call(c, cuda_device, path="tc")
    ops.check_status(cuda_device)
    assert_within(got, want, *TOL[torch.bfloat16], what=f"tc tile~{tile}")
    simt = call(c, cuda_device, path="simt")
    assert_within(got, simt, 1e-2, 1e-2, what="tc vs simt")
    assert torch.equal(got, call(c, cuda_device, path="tc"))


def test_tensor_core_path_refuses_unfit_shapes(cuda_device):
    c = load_case("int4_sweep2")  # K=96, N=48
    with pytest.raises(RuntimeError, match="tcgen05"):
        call(c, cuda_device, path="tc")


def test_golden_no_routed_weight(cuda_device):
    c = load_case("int4_tiny")
    out = call(c, cuda_device, mul_routed_weight=False)
    assert_within(out, load_case("int4_tiny_noweight")["out"], *TOL[torch.bfloat16], what="noweight")


def test_golden_replicated_expert_parallel(cuda_device):
    c = load_case("int4_tiny")
    total = torch.zeros(c["out"].shape, dtype=torch.float32)
    for rank in range(2):
        g = load_case(f"int4_tiny_ep_rank{rank}")
        sl = slice(rank * 4, (rank + 1) * 4)
        d = to_dev({k: c[k] for k in KEYS}, cuda_device)
        part = xkb.fused_moe_int4_w4a16(d["A"], d["packed"][sl].contiguous(), d["scale"][sl].contiguous(),
                                        d["topk_ids"], d["topk_w"], expert_map=g["expert_map"].to(cuda_device))
        assert_within(part, g["out"], *TOL[torch.bfloat16], what=f"partial rank {rank}")
        total += part.float().cpu()
    assert_within(total, c["out"].float(), 2e-2, 2e-2, what="sum of partials")


@pytest.mark.parametrize("M,K,N,E,top_k,group,dtype", [
    (16, 64, 32, 4, 2, 32, torch.bfloat16), (1, 64, 32, 4, 2, 32, torch.bfloat16),
    (37, 96, 48, 8, 3, 32, torch.bfloat16), (16, 64, 32, 4, 2, 32, torch.float32),
    (5, 128, 130, 3, 2, 64, torch.bfloat16), (9, 256, 17, 2, 1, 128, torch.float32),
    (33, 512, 256, 6, 4, 32, torch.bfloat16), (3, 40, 8, 2, 2, 8, torch.bfloat16),
])
def test_against_oracle_with_repeated_ids(M, K, N, E, top_k, group, dtype, cuda_device):
    """Harness-style inputs (registry/input_gen.py:138-159): ids drawn with replacement, weights
    uniform and not normalised."""
    g = torch.Generator().manual_seed(M * 7 + K)
    A = torch.randn(M, K, generator=g).to(dtype)
    codes = torch.randint(0, 16, (E, N, K), generator=g)
    packed = synth.pack_int4_codes(codes)
    scale = (torch.rand(E, N, K // group, generator=g) * 0.02 + 0.005).to(torch.bfloat16)
    ids = torch.randint(0, E, (M, top_k), generator=g, dtype=torch.int32)
    w = torch.rand(M, top_k, generator=g)
    want = oracle.moe_w4a16_loop(A, packed, scale, ids, w, group)
    c = {"A": A, "packed": packed, "scale": scale, "topk_ids": ids, "topk_w": w, "group_size": group}
    got = call(c, cuda_device)
    assert_within(got, want, *TOL[dtype], what="auto")
    assert torch.equal(got, call(c, cuda_device)), "second run differs: the combine must be deterministic"


def test_padding_never_leaks(cuda_device):
    """Poisoned activations for tokens that no slot of a hot expert uses must not reach other
    rows: NaN in one token's row only shows up in that token's output row."""
    c = load_case("int4_tiny")
    A = c["A"].clone()
    A[3] = float("nan")
    c2 = dict(c, A=A)
    out = call(c2, cuda_device).cpu()
    assert torch.isnan(out[3]).all()
    keep = [i for i in range(out.shape[0]) if i != 3]
    assert_within(out[keep], c["out"][keep], *TOL[torch.bfloat16], what="other rows")


def test_decode_config_full_output_and_properties(cuda_device):
    """M=64, K=7168, N=4096, E=48, top_k=8 at full size: all 64 x 4096 outputs against the oracle
    (about 15 s of CPU), then determinism and linearity in the routing weights."""
    cfg = synth.CONFIGS["int4_decode"]
    d = synth.make_int4(cfg, seed=1729, device=cuda_device)
    out = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])
    assert out.shape == (cfg.M, cfg.N) and out.dtype == torch.bfloat16
    want = oracle.moe_w4a16(d["A"].cpu(), d["packed"].cpu(), d["scale"].cpu(), d["topk_ids"].cpu(),
                            d["topk_w"].cpu(), 32)
    assert_within(out, want, *TOL[torch.bfloat16], what="decode, all columns")
    assert torch.equal(out, xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"]))
    out2 = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], 2 * d["topk_w"])
    assert_within(out2.float(), 2 * out.float(), 1.6e-2, 1e-2, what="linearity in topk_w")


@pytest.mark.parametrize("M", [1, 64])
def test_down_projection_shape_against_oracle(M, cuda_device):
    """The second expert-GEMM shape of the reference's INT4 benchmark (N=7168, K=2048, E=48, top_k=8:
    meta/benchmarks/bench_moe_int4_w4a16.py:8-12,90-91), where a tile is only eight 256-K stages
    long: the whole output against the oracle."""
    from xkernels_b200 import ops

    cfg = synth.Int4Config("down", M=M, K=2048, N=7168, E=48, top_k=8)
    d = synth.make_int4(cfg, seed=77, device=cuda_device)
    out = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])
    ops.check_status(cuda_device)
    want = oracle.moe_w4a16(d["A"].cpu(), d["packed"].cpu(), d["scale"].cpu(), d["topk_ids"].cpu(), d["topk_w"].cpu(), 32)
    assert_within(out, want, *TOL[torch.bfloat16], what=f"down projection shape, M={M}")


def test_alternating_shapes_share_the_workspace(cuda_device):
    """Calls of different shapes take turns on the per-device workspace, so the routing of one call
    lies where the other call keeps slot rows or activations.  The kernels of a call overlap
    (programmatic dependent launch): one that read the routing before the align stage of ITS call
    had written it would see the other call's bytes there.  Every call must reproduce its first
    result bit for bit and leave the status word clear."""
    from xkernels_b200 import ops

    cfgs = [synth.Int4Config("a", M=64, K=2048, N=7168, E=48, top_k=8),
            synth.Int4Config("b", M=1, K=2048, N=7168, E=48, top_k=8),
            synth.Int4Config("c", M=40, K=1024, N=512, E=16, top_k=4)]
    data = [synth.make_int4(c, seed=70 + i, device=cuda_device) for i, c in enumerate(cfgs)]
    call = lambda d: xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])  # noqa: E731
    first = []
    for d in data:
        first.append(call(d))
        ops.check_status(cuda_device)
    for _round in range(8):
        for d, want in zip(data, first):
            got = call(d)
            ops.check_status(cuda_device)
            assert torch.equal(got, want)


def test_prefill_sized_batch_whole_output(cuda_device):
    """16 384 slots at 128-token tiles (two row tiles per token tile), skewed routing: the whole
    output against the oracle, repeated calls bit-identical, status clear."""
    from xkernels_b200 import ops

    cfg = synth.Int4Config("prefill_sized", M=2048, K=1024, N=512, E=16, top_k=8, expert_bias_std=0.5)
    d = synth.make_int4(cfg, seed=5, device=cuda_device)
    out = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"], path="tc")
    ops.check_status(cuda_device)
    want = oracle.moe_w4a16(d["A"].cpu(), d["packed"].cpu(), d["scale"].cpu(), d["topk_ids"].cpu(), d["topk_w"].cpu(), 32)
    assert_within(out, want, *TOL[torch.bfloat16], what="prefill-sized batch")
    for _ in range(5):
        again = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"], path="tc")
        ops.check_status(cuda_device)
        assert torch.equal(out, again)


def prefill_token_sample(topk_ids: torch.Tensor, E: int, block: int, n_tokens: int, seed: int) -> torch.Tensor:
    """Token rows to check at the prefill configuration: for every expert the tokens whose slots sit
    at the first and the last position of the expert's sorted run (so the first and the last,
    partly padded, token block of every expert are hit), filled up with random tokens."""
    sorted_ids, _expert_ids, num_post = oracle.align_block_size(topk_ids.numpy(), block, E)
    top_k = topk_ids.shape[1]
    numel = topk_ids.numel()
    counts = torch.bincount(topk_ids.reshape(-1).long(), minlength=E).tolist()
    picked, pos = [], 0
    for e in range(E):
        if counts[e]:
            picked += [int(sorted_ids[pos]) // top_k, int(sorted_ids[pos + counts[e] - 1]) // top_k]
        pos += -(-counts[e] // block) * block
    assert pos == int(num_post[0]) and all(0 <= t * top_k < numel for t in picked)
    g = torch.Generator().manual_seed(seed)
    extra = torch.randperm(topk_ids.shape[0], generator=g).tolist()
    seen = set(picked)
    for t in extra:
        if len(seen) >= n_tokens:
            break
        seen.add(t)
    return torch.tensor(sorted(seen), dtype=torch.long)


def test_prefill_config_token_sample_against_oracle(cuda_device):
    """M=16384, K=7168, N=4096, E=48, top_k=8 with the skewed router at full size (the 128-token
    row-tile-pair mode of the tcgen05 kernel).  The reference loop is infeasible at this size
    (131 072 Python iterations, ops/moe/reference.py:54-70), so 256 token rows x all 4096 columns
    are compared with the oracle run on exactly those tokens: every expert is hit, in the first
    and in the last token block of its run.  The whole output is checked through determinism."""
    from xkernels_b200 import ops

    cfg = synth.CONFIGS["int4_prefill"]
    d = synth.make_int4(cfg, seed=1729, device=cuda_device)
    out = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])
    ops.check_status(cuda_device)
    assert out.shape == (cfg.M, cfg.N) and out.dtype == torch.bfloat16
    ids_cpu = d["topk_ids"].cpu()
    sel = prefill_token_sample(ids_cpu, cfg.E, 128, 256, seed=3)
    assert sel.numel() >= 256 and torch.unique(ids_cpu[sel]).numel() == torch.unique(ids_cpu).numel()
    want = oracle.moe_w4a16(d["A"][sel.to(cuda_device)].cpu(), d["packed"].cpu(), d["scale"].cpu(), ids_cpu[sel],
                            d["topk_w"].cpu()[sel], 32)
    assert_within(out[sel.to(cuda_device)], want, *TOL[torch.bfloat16], what="prefill token sample")
    assert bool(torch.isfinite(out.float()).all())
    again = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])
    assert torch.equal(out, again)


@pytest.mark.parametrize("path", ["simt", "tc"])
@pytest.mark.parametrize("with_map", [False, True])
def test_slots_without_a_local_expert_are_dropped(path, with_map, cuda_device):
    """Ids of -1 ("no expert") and ids >= E (global ids against rank-local weights) contribute
    nothing, with and without an expert_map: the align stage drops the slot and the combine must
    skip its never-written fp32 row (the reference skips such slots, ops/moe/reference.py:59-63 with
    a map, ops/moe/mxfp4_reference.py:82-83 without).  The workspace is poisoned first so that a
    stale row would show."""
    from xkernels_b200 import ops

    cfg = synth.Int4Config("drop", M=40, K=512, N=256, E=6, top_k=4)
    c = synth.make_int4(cfg, seed=31)
    g = torch.Generator().manual_seed(9)
    ids = c["topk_ids"].clone()
    kill = torch.rand(cfg.M, cfg.top_k, generator=g)
    ids[kill < 0.2] = -1
    ids[(kill >= 0.2) & (kill < 0.4)] = cfg.E + 3
    ids[0] = -1                                           # a token with no expert at all -> zero row
    if with_map:
        emap = torch.arange(cfg.E + 8, dtype=torch.int32)
        emap[cfg.E:] = -1
        emap[2] = -1                                      # and one real expert that is "elsewhere"
    else:
        emap = None
    # oracle: the same routing with every dropped slot sent through a map entry of -1
    drop = (ids < 0) | (ids >= cfg.E) | ((ids == 2) if with_map else torch.zeros_like(ids, dtype=torch.bool))
    o_ids = torch.where(drop, torch.full_like(ids, cfg.E), ids)
    o_map = torch.cat([torch.arange(cfg.E, dtype=torch.int32), torch.tensor([-1], dtype=torch.int32)])
    want = oracle.moe_w4a16(c["A"], c["packed"], c["scale"], o_ids, c["topk_w"], 32, expert_map=o_map)
    d = to_dev(c, cuda_device)
    ws_bytes = 1 << 24
    ops.get_workspace(cuda_device, ws_bytes).view(torch.float32)[64:].fill_(1.0e4)   # stale rows would be huge
    got = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], ids.to(cuda_device), d["topk_w"],
                                   expert_map=None if emap is None else emap.to(cuda_device), path=path)
    ops.check_status(cuda_device)
    assert_within(got, want, *TOL[torch.bfloat16], what=f"dropped slots/{path}/map={with_map}")
    assert bool((got[0] == 0).all())


def test_cpu_tensor_is_refused():
    c = load_case("int4_sweep0")
    with pytest.raises(RuntimeError, match="CUDA"):
        xkb.fused_moe_int4_w4a16(c["A"], c["packed"], c["scale"], c["topk_ids"], c["topk_w"])


@pytest.mark.parametrize("E,per_expert,N", [(32, 8, 128), (32, 16, 128), (32, 32, 128), (2, 256, 256), (2, 256, 128)])
def test_dequantised_weights_are_bit_exact(E, per_expert, N, cuda_device):
    """The in-kernel dequantiser against ``dequant_w4a16`` (src/xkernels/ops/moe/w4a16.py:21-50), bit
    for bit, through the tcgen05 GEMM: one-hot activations (1.0 at one k), top_k = 1 and routing
    weight 1 make ``out[token] = W[expert][:, k]`` with nothing to round but the weight itself.
    Every k position of a 256-K stage, every nibble value, scales from 2^-20 to 2^10 (both signs)
    and zero scales are covered, at every token-tile width of the kernel."""
    from xkernels_b200 import ops

    K = 256
    g = torch.Generator().manual_seed(E * 1000 + per_expert)
    codes = torch.randint(0, 16, (E, N, K), generator=g)
    codes[:, :16, :] = torch.arange(16).view(1, 16, 1)           # every nibble value at every position
    packed = synth.pack_int4_codes(codes)
    expo = torch.randint(-20, 11, (E, N, K // 32), generator=g).float()
    mant = 1.0 + torch.rand(E, N, K // 32, generator=g)
    sign = torch.where(torch.rand(E, N, K // 32, generator=g) < 0.3, -1.0, 1.0)
    scale = (sign * mant * torch.exp2(expo)).to(torch.bfloat16)
    scale[:, 5, :] = 0.0
    want_w = oracle.dequant_w4a16(packed, scale, 32, out_dtype=torch.bfloat16)      # [E, N, K]
    M = E * per_expert
    ids = torch.arange(E, dtype=torch.int32).repeat_interleave(per_expert).view(M, 1)
    ones = torch.ones(M, 1)
    n_rounds = K // per_expert if per_expert < K else 1
    for r in range(n_rounds):
        ks = (torch.arange(M) % per_expert) + r * per_expert                       # k probed by each token
        A = torch.zeros(M, K, dtype=torch.bfloat16)
        A[torch.arange(M), ks] = 1.0
        out = xkb.fused_moe_int4_w4a16(A.to(cuda_device), packed.to(cuda_device), scale.to(cuda_device),
                                       ids.to(cuda_device), ones.to(cuda_device), path="tc").cpu()
        ops.check_status(cuda_device)
        want = want_w[ids.view(-1).long(), :, ks]                                   # [M, N]
        assert torch.equal(out, want), f"round {r}: {(out != want).sum().item()} dequantised weights differ"
