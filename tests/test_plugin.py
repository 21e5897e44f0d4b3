"""The plug-in boundary on CPU: cards validate against the reference's own schema, the overlay
registry loads, find_impl lists the sm_100 cards, and a CUDA card on CPU tensors is a clean
"not runnable" (RuntimeError) instead of a crash.  Skipped where no copy of the reference exists."""

import json
from pathlib import Path

import pytest

from tests.reference_util import reference_available

ROOT = Path(__file__).resolve().parents[1]
HAVE_REF = reference_available(allow_source_tree=True)
needs_ref = pytest.mark.skipif(not HAVE_REF, reason="reference package not available")


def test_overlay_files_are_well_formed():
    reg = ROOT / "xkernels_b200" / "registry"
    cards = sorted((reg / "impls").glob("*.card.json"))
    assert len(cards) == 6
    for c in cards:
        doc = json.loads(c.read_text())
        assert c.name == f"{doc['implements'].split('@')[0]}.{doc['backend']}.card.json"
        if doc["backend"] == "cuda":
            assert doc["arch"]["family"] == "nvidia_sm100" and doc["arch"]["wave_size"] == 32
            for m in doc["perf"]["measured"]:
                assert m["source"] and m["arch"] == "nvidia_sm100"
    sweep = json.loads((reg / "shape_sweeps" / "moe_mxfp4.sweep.json").read_text())
    assert len(sweep["points"]) >= 3 and any(p["dtype"] == "fp32" for p in sweep["points"])


@needs_ref
def test_install_registers_cards_and_backends(tmp_path):
    from xkernels_b200 import plugin

    root = plugin.install(tmp_path / "overlay")
    from xkernels._backends import Backend
    from xkernels._dispatch import registered_backends
    from xkernels.registry import loader

    for k in plugin.KERNELS:
        assert Backend.CUDA in registered_backends(k)
    for cid in plugin.CARD_IDS:
        card = loader.get_card(cid)
        assert card.implements.split("@")[0] == cid.split(".")[0]
    assert loader.get_spec("moe_mxfp4@1.0.0").kernel == "moe_mxfp4"
    assert len(loader.load_shape_sweep("moe_mxfp4")) >= 3
    assert (Path(root) / "impls" / "moe_sum_reduce.cuda.card.json").exists()


@needs_ref
def test_find_impl_lists_the_sm100_cards(tmp_path):
    from xkernels_b200 import plugin

    plugin.install(tmp_path / "overlay")
    from xkernels import find_impl

    found = find_impl("gemm", target_arch="nvidia_sm100")
    text = json.dumps(found, default=str)
    assert "moe_int4_w4a16.cuda@1.0.0" in text
    assert "moe_align_block_size.cuda@1.0.0" in json.dumps(find_impl("scatter", target_arch="nvidia_sm100"), default=str)
    assert "moe_sum_reduce.cuda@1.1.0" in json.dumps(find_impl("reduce", target_arch="nvidia_sm100"), default=str)


@needs_ref
def test_reference_cards_verify_and_cuda_is_not_runnable_on_cpu(tmp_path):
    from xkernels_b200 import plugin

    plugin.install(tmp_path / "overlay")
    from xkernels import verify, verify_parity

    res = verify("moe_mxfp4.reference@1.0.0")
    assert res["correctness"]["passed"] is True
    par = verify_parity("moe_int4_w4a16@1.0.0")          # device defaults to cpu: our card cannot run there
    assert par["inconclusive"] is True and par["n_runnable"] == 1
    par = verify_parity("moe_mxfp4@1.0.0")
    assert par["n_runnable"] == 1


@needs_ref
def test_cards_validate_against_the_reference_schema_and_write_back_goes_through_its_function(tmp_path):
    """Every card of this package passes the reference's impl_card schema (the optional `persistent`
    block included, registry/schema/impl_card.schema.json:169-222), and plugin.write_back records a
    measurement with the reference's own record_measurement: sourced, replacing the same point."""
    import jsonschema
    import xkernels

    from xkernels_b200 import plugin

    plugin.install(tmp_path / "overlay")
    from xkernels.registry import schemas

    schema = json.loads((Path(schemas._SCHEMA_DIR) / "impl_card.schema.json").read_text())
    cards = sorted((ROOT / "xkernels_b200" / "registry" / "impls").glob("*.card.json"))
    for c in cards:
        jsonschema.validate(json.loads(c.read_text()), schema)
    tc = json.loads((ROOT / "xkernels_b200" / "registry" / "impls" / "moe_int4_w4a16.cuda.card.json").read_text())
    assert tc["persistent"]["tensor_memory_columns"] == 512 and tc["arch"]["scratch"]["bytes"] > 100000
    assert any("dequantiser" in r for r in tc["persistent"]["warp_roles"])

    out = tmp_path / "cards"
    shape = {"M": 64, "K": 7168, "N": 4096, "E": 48, "top_k": 8}
    plugin.write_back("moe_int4_w4a16.cuda@1.0.0", shape=shape, dtype="bf16", source="run:test#1", ms=0.25,
                      achieved_bw_pct=50.0, cards_dir=out)
    plugin.write_back("moe_int4_w4a16.cuda@1.0.0", shape=shape, dtype="bf16", source="run:test#2", ms=0.2,
                      achieved_bw_pct=62.0, cards_dir=out)
    doc = json.loads((out / "moe_int4_w4a16.cuda.card.json").read_text())
    jsonschema.validate(doc, schema)
    same = [m for m in doc["perf"]["measured"] if m["shape"] == shape]
    assert len(same) == 1 and same[0]["source"] == "run:test#2" and same[0]["ms"] == 0.2
    with pytest.raises(ValueError):
        plugin.write_back("moe_int4_w4a16.cuda@1.0.0", shape=shape, dtype="bf16", source="", ms=0.2, cards_dir=out)
    assert xkernels is not None
