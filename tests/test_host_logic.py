"""Host-side logic of the package that needs no GPU."""
import os

import pytest
import torch

from vui_b200.engine import GenConfig, _get_bucket, _make_buckets
from vui_b200.model import VuiShape, freqs_cis_table, state_dict_shapes
from vui_b200.text import chunk_text, simple_clean


def test_shape_facts():
    s = VuiShape()
    assert s.rq_ffn == 1408  # RQBlock computes 64*ceil(int(512*8/3)/64)
    assert s.head_dim == 64
    assert VuiShape(max_secs=30).max_seq_len == 1344 + 16
    shapes = state_dict_shapes(s)
    assert shapes["rq_transformer.blocks.0.w1.weight"] == (1408, 512)
    assert shapes["decoder.blocks.23.attn.Wqkv.weight"] == (2048, 1024)
    n = sum(torch.Size(v).numel() for v in shapes.values())
    assert 530e6 < n < 545e6


def test_product_and_oracle_agree_on_names_and_init():
    from oracle.vui_oracle import OracleConfig, weight_shapes

    assert weight_shapes(OracleConfig()) == state_dict_shapes(VuiShape())


def test_rope_table_matches_reference_rows(golden_dir):
    fx = torch.load(os.path.join(golden_dir, "ops_bf16.pt"))
    t = freqs_cis_table(64, 1360, 1e6).to(torch.bfloat16)
    assert torch.equal(t[fx["rope_pos"]], fx["rope_table_rows"])


def test_buckets():
    assert _make_buckets(1) == [1]
    assert _make_buckets(8) == [1, 2, 4, 8]
    assert _make_buckets(6) == [1, 2, 4, 6]
    assert _get_bucket(3, [1, 2, 4, 8]) == 4
    assert _get_bucket(9, [1, 2, 4, 8]) == 8


def test_max_turn_frames():
    c = GenConfig()
    assert c.max_turn_frames(0) == int(15.0 * 12.5)
    assert c.max_turn_frames(5) == int((5 / 3.0 * 1.6 + 0.6) * 12.5)
    assert c.max_turn_frames(5, prompt_wps=2.0) == int((5 / 2.0 * 1.6 + 0.6) * 12.5)
    assert GenConfig(max_turn_wps=4.0).max_turn_frames(8, 2.0) == int((8 / 4.0 * 1.6 + 0.6) * 12.5)
    assert c.max_turn_frames(1000) == 187


def test_text_against_reference_fixture(golden_dir):
    import json

    with open(os.path.join(golden_dir, "text_cases.json")) as f:
        cases = json.load(f)
    for c in cases["clean"]:
        assert simple_clean(c["in"]) == c["out"], c["in"]
    for c in cases["chunk"]:
        assert chunk_text(c["in"], **c["kw"]) == c["out"], (c["in"], c["kw"])


def test_engine_refuses_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("has CUDA")
    from vui_b200 import Engine

    with pytest.raises(RuntimeError):
        Engine(model=None)
