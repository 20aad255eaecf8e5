"""GraphedModule: a captured forward call replays to the same bits as the eager call, for new input values too."""

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def test_graphed_diffusion_stack_equals_eager(pkg):
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    n = 40
    g = torch.Generator().manual_seed(5)
    model = pkg.DiffusionTransformer(**cases.DIFF, no_blocks=2, use_ada_layer_norm=True, n_query=None, n_key=None,
                                     inf=1e9)
    model.load_state_dict(pkg.weights.diffusion_stack_params(seed=21, no_blocks=2, **cases.DIFF), strict=True)
    model = model.to(dev, bf).eval()
    model.hoist_pair_bias = False

    def draw():
        a = torch.randn(1, 3, n, 768, generator=g).to(dev, bf)
        s = torch.randn(1, 3, n, 384, generator=g).to(dev, bf)
        z = torch.randn(1, 1, n, n, 128, generator=g).to(dev, bf)
        m = torch.ones(1, 1, n, dtype=bf, device=dev)
        m[..., -5:] = 0
        return a, s, z, m

    fn = lambda a, s, z, m: model(a, s, z, mask=m)
    first = draw()
    graphed = pkg.GraphedModule(fn, *first)
    with torch.no_grad():
        for x in (first, draw(), tuple(t.cpu().pin_memory() for t in draw())):
            want = fn(*(t.to(dev) for t in x))
            got = graphed(*x)
            torch.cuda.synchronize()
            assert torch.equal(got, want)
    pkg.lib.check_device_status()
    with pytest.raises(ValueError):
        graphed(first[0][:, :2], *first[1:])


def test_graphed_pairformer_stack_equals_eager(pkg):
    """The trunk's forward uses two streams (the single track runs beside the next block's pair stack): the capture
    must take both, and the in-place update of the captured input buffers must not leak into the next call."""
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    n = 64
    g = torch.Generator().manual_seed(6)
    stack = pkg.PairFormerStack(**cases.OF3, no_blocks=3, blocks_per_ckpt=None, transition_type="swiglu",
                                pair_dropout=0.25, fuse_projection_weights=False, inf=1e9)
    stack.load_state_dict(pkg.weights.pairformer_stack_params(seed=22, no_blocks=3, **cases.OF3), strict=True)
    stack = stack.to(dev, bf).eval()

    def draw():
        s = torch.randn(1, n, 384, generator=g).to(dev, bf)
        z = torch.randn(1, n, n, 128, generator=g).to(dev, bf)
        sm = cases.rand_mask((1, n), g).to(dev, bf)
        pm = cases.token_pair_mask(sm.float().cpu()).to(dev, bf)
        return s, z, sm, pm

    fn = lambda s, z, sm, pm: stack(s, z, sm, pm, inplace_safe=True)
    first = draw()
    graphed = pkg.GraphedModule(fn, *first)
    with torch.no_grad():
        for x in (first, draw(), first):
            want = stack(*x)   # clones its inputs
            got = graphed(*x)
            torch.cuda.synchronize()
            assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    pkg.lib.check_device_status()
