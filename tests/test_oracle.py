"""CPU tests: the oracle against fixtures produced by the reference's own code."""
import pytest
import torch

import attention_oracle as orc
from _util import golden_case_names, load_config1_head, load_golden


@pytest.mark.parametrize("name", golden_case_names())
def test_mask_matches_reference(name):
    meta, _, _, mask = load_golden(name)
    m = orc.visibility_mask(meta["chunk_id"], meta["N_q"], meta["N_kv"], meta["window_size"])
    assert torch.equal(m, mask)
    assert orc.visible_pairs(meta["chunk_id"], meta["N_q"], meta["N_kv"],
                             meta["window_size"]) == int(mask.sum())


@pytest.mark.parametrize("name", golden_case_names())
def test_autograd_oracle_matches_reference(name):
    meta, inp, out, mask = load_golden(name)
    got = orc.autograd_all(*(inp[n] for n in orc.INPUT_NAMES), mask)
    for n in orc.OUTPUT_NAMES:
        ref = out[n]
        g = torch.nan_to_num(got[n].float(), neginf=float("-inf"))
        if n == "L":   # fully masked rows hold -inf on both sides
            assert torch.equal(torch.isinf(g), torch.isinf(ref))
            g, ref = torch.nan_to_num(g, neginf=0.0), torch.nan_to_num(ref, neginf=0.0)
        assert torch.allclose(g, ref, rtol=1e-6, atol=1e-6), n


@pytest.mark.parametrize("name", golden_case_names())
def test_closed_form_matches_reference(name):
    meta, inp, out, _ = load_golden(name)
    got = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES),
                              window_size=meta["window_size"], chunk_id=meta["chunk_id"],
                              row_block=48)
    for n in orc.OUTPUT_NAMES:
        ref = torch.nan_to_num(out[n], neginf=0.0)
        g = torch.nan_to_num(got[n].float(), neginf=0.0)
        assert orc.max_abs_err(g, ref) <= 1e-5 * max(1.0, float(ref.abs().max())), n


def test_config1_head_and_norms():
    (b, h), inp, out, norms, sums = load_config1_head()
    # regenerate the full config from its seed: the stored head must be a slice of it
    full = orc.make_inputs(2, 4, 256, 256, 64, seed=0, dtype=torch.float32)
    for n in orc.INPUT_NAMES:
        assert torch.equal(full[n][b, h], inp[n]), n
    mask = orc.visibility_mask(0, 256, 256, 256)
    assert torch.equal(mask, torch.ones(256, 256, dtype=torch.bool).tril())
    got = orc.closed_form_all(*(full[n] for n in orc.INPUT_NAMES), window_size=256, chunk_id=0)
    for n in orc.OUTPUT_NAMES:
        assert orc.rel_err(got[n][b, h], out[n]) < 1e-6, n
        assert abs(float(got[n].double().norm()) - norms[n]) <= 1e-9 * norms[n], n
    one = {n: full[n][b:b + 1, h:h + 1] for n in orc.INPUT_NAMES}
    ag = orc.autograd_all(*(one[n] for n in orc.INPUT_NAMES), mask)
    for n in orc.OUTPUT_NAMES:
        assert orc.rel_err(ag[n][0, 0], out[n]) < 1e-6, n


def test_mask_none_and_visible_pairs():
    m = orc.visibility_mask(0, 5, 9, 3, orc.MASK_NONE)
    assert bool(m.all()) and orc.visible_pairs(0, 5, 9, 3, orc.MASK_NONE) == 45
    for (cid, nq, nkv, ws) in [(0, 64, 64, 64), (0, 64, 64, 7), (2, 32, 128, 96), (0, 96, 40, 1000),
                               (1, 72, 200, 150), (0, 4096, 4096, 4096)]:
        if nq * nkv <= 1 << 22 or True:
            assert orc.visible_pairs(cid, nq, nkv, ws) == int(orc.visibility_mask(cid, nq, nkv, ws).sum())
    assert orc.visible_pairs(0, 4096, 4096, 4096) == 4096 * 4097 // 2
