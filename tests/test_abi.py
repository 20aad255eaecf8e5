"""The C-ABI library: builds for sm_100a, loads without a GPU, exports every symbol the public
header declares, and rejects bad arguments with error codes instead of crashing."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "of3b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(of3_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "of3_trimul_forward" in syms and "of3_triattn_forward" in syms and len(syms) >= 15


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.lib.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/of3b200.h but not exported"
    assert set(pkg.lib.SIGNATURES) == set(declared_symbols())


def test_bad_arguments_return_error_codes(pkg):
    lib = pkg.lib.load()
    p = pkg.lib.TrimulParams()
    rc = lib.of3_trimul_forward(None, None, None, 1, 8, 128, 128, 0, 0, ctypes.byref(p), None, 0, None)
    assert rc == -1 and b"null" in lib.of3_last_error_string()
    rc = lib.of3_trimul_forward(None, None, None, 1, 8, 128, 128, 7, 0, ctypes.byref(p), None, 0, None)
    assert rc == -1 and b"dtype" in lib.of3_last_error_string()
    t = pkg.lib.TransitionParams()
    assert lib.of3_transition_forward(None, None, None, 4, 128, 4, 1, 0, ctypes.byref(t), None, 0, None) == -1


def test_workspace_queries_need_no_gpu(pkg):
    lib = pkg.lib.load()
    for dt in (0, 1):
        assert lib.of3_trimul_workspace_bytes(1, 64, 128, 128, dt, 0) > 0
        assert lib.of3_triattn_workspace_bytes(1, 64, 128, 4, 32, dt, 0) > 0
        assert lib.of3_transition_workspace_bytes(4096, 128, 4, dt, 0) > 0
        assert lib.of3_attn_pair_bias_workspace_bytes(2, 1, 64, 384, 0, 128, 16, 24, dt, 0) > 0
        assert lib.of3_cond_transition_workspace_bytes(128, 768, 384, 2, dt, 0) > 0


def test_no_cpu_fallback(pkg):
    """CPU tensors are refused: there is no path that avoids the CUDA library."""
    m = pkg.TriangleMultiplicationOutgoing(128, 128).eval()
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.zeros(1, 4, 4, 128))


def test_forward_only(pkg):
    m = pkg.SwiGLUTransition(128, 4)
    with pytest.raises(NotImplementedError):
        m(torch.zeros(1, 4, 128, requires_grad=True))


def test_state_dict_keys_match_reference_layout(pkg):
    P = pkg.weights.pairformer_block_params(1)
    blk = pkg.PairFormerBlock(c_s=384, c_z=128, c_hidden_pair_bias=24, no_heads_pair_bias=16,
                              c_hidden_mul=128, c_hidden_pair_att=32, no_heads_pair=4,
                              transition_type="swiglu", transition_n=4, pair_dropout=0.25,
                              fuse_projection_weights=False, inf=1e9)
    assert len(P) == 57 and sum(v.numel() for v in P.values()) == 3070848
    blk.load_state_dict(P, strict=True)
    # a freshly constructed block is the identity on (s, z): its zero-initialised matrices
    zeros = [k for k, v in blk.state_dict().items() if v.abs().sum() == 0 and v.dim() == 2]
    assert len(zeros) == 0  # we just loaded random weights
    fresh = pkg.PairFormerBlock(c_s=384, c_z=128, c_hidden_pair_bias=24, no_heads_pair_bias=16,
                                c_hidden_mul=128, c_hidden_pair_att=32, no_heads_pair=4,
                                transition_type="swiglu", transition_n=4, pair_dropout=0.25,
                                fuse_projection_weights=False, inf=1e9)
    zeros = [k for k, v in fresh.state_dict().items() if v.dim() == 2 and v.abs().sum() == 0]
    assert len(zeros) == 16


def test_modules_pack_grouped_weights_back_to_back(pkg):
    """Linear layers that share an input run as one launch when their weights lie back to back in memory (the
    library compares addresses): the modules' parameter packer must lay q | g | k | v, the AdaLN pair and the
    SwiGLU pair out that way, with unchanged values."""
    dt, dev = torch.bfloat16, torch.device("cpu")
    apb = pkg.AttentionPairBias(c_q=768, c_k=768, c_v=768, c_s=384, c_z=128, c_hidden=48, no_heads=16,
                                use_ada_layer_norm=True, inf=1e9)
    prm = apb._params(dt, dev)
    step = 768 * 768 * 2
    q, g, k, v = prm[11], prm[15], prm[13], prm[14]
    assert [t.data_ptr() - q.data_ptr() for t in (g, k, v)] == [step, 2 * step, 3 * step]
    assert torch.equal(q, apb.mha.linear_q.weight.to(dt)) and torch.equal(v, apb.mha.linear_v.weight.to(dt))
    assert torch.equal(g, apb.mha.linear_g.weight.to(dt)) and torch.equal(k, apb.mha.linear_k.weight.to(dt))
    assert prm[5].data_ptr() - prm[3].data_ptr() == 768 * 384 * 2          # AdaLN linear_g, linear_s
    ctb = pkg.ConditionedTransitionBlock(c_a=768, c_s=384, n=2)
    prm = ctb._params(dt, dev)
    assert prm[3].data_ptr() - prm[1].data_ptr() == 768 * 384 * 2          # AdaLN pair
    assert prm[5].data_ptr() - prm[4].data_ptr() == 2 * 768 * 768 * 2      # SwiGLU linear_a, linear_b
    tr = pkg.SwiGLUTransition(c_in=384, n=4)
    prm = tr._params(dt, dev)
    assert prm[3].data_ptr() - prm[2].data_ptr() == 4 * 384 * 384 * 2
    assert torch.equal(prm[3], tr.swiglu.linear_b.weight.to(dt))
