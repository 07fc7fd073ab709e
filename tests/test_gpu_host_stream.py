"""The host-buffer entry point (``ops3d_b200.host_stream``): inputs and outputs in host memory, the step cut
into query chunks that upload, compute and download concurrently.  It must give what the one-shot operator
gives on device tensors -- ``out`` and ``grad_packed`` rows bit for bit (rows are independent), ``grad_value``
up to the order of the fp32 atomics -- and agree with the CPU oracle."""
import pytest
import torch

from oracle import fda_oracle
from ops3d_b200 import capi
from ops3d_b200.host_stream import HostStreamedStep, flash_deform_attn_host

pytestmark = pytest.mark.gpu


def _one_shot(value, sh, lsi, packed, grad_out, K, dev="cuda"):
    v, pk, go = value.to(dev), packed.to(dev), grad_out.to(dev)
    out = capi.forward(v, sh.to(dev), lsi.to(dev), pk, K)
    gv, gp = capi.backward(v, sh.to(dev), lsi.to(dev), pk, go, K)
    torch.cuda.synchronize()
    return out.cpu(), gv.cpu(), gp.cpu()


@pytest.mark.parametrize("vdt,pdt", [(torch.bfloat16, torch.float32), (torch.float32, torch.float32),
                                     (torch.float16, torch.float16)])
@pytest.mark.parametrize("chunk", [37, 64, 1000])
def test_chunked_host_step_equals_one_shot(vdt, pdt, chunk):
    shapes = [(6, 8, 10), (3, 4, 5)]
    B, Q, G, D, K = 2, 150, 4, 32, 4
    value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(shapes, B, Q, G, D, K, seed=41)
    value_h, packed_h, go_h = value.to(vdt).pin_memory(), packed.to(pdt).pin_memory(), grad_out.to(vdt).pin_memory()
    want_out, want_gv, want_gp = _one_shot(value_h, sh, lsi, packed_h, go_h, K)
    got_out, got_gv, got_gp = flash_deform_attn_host(value_h, sh, lsi, packed_h, go_h, K, chunk_queries=chunk)
    assert torch.equal(got_out, want_out)
    assert torch.equal(got_gp, want_gp)
    tol = 1e-4 if vdt == torch.float32 else 2e-2
    ref_out, ref_gv, ref_gp = fda_oracle.fused_forward_backward(value_h, sh, packed_h, go_h, K)
    scale = max(1.0, ref_gv.abs().max().item())
    assert (got_gv.float() - want_gv.float()).abs().max().item() <= tol * scale
    assert (got_gv.float() - ref_gv).abs().max().item() <= tol * scale
    assert (got_out.float() - ref_out).abs().max().item() <= tol * max(1.0, ref_out.abs().max().item())


def test_step_object_is_reusable_and_counts_its_copies(fda_env):
    """Same object, two runs with different data (slots and events are reused); slab-binned path forced on."""
    fda_env(FDA_L2_KEEP_FRACTION="0.00001", FDA_BIN_SLAB_MB="0.05")
    shapes = [(8, 6, 10), (4, 3, 5)]
    B, Q, G, D, K = 2, 90, 4, 32, 8
    dev = torch.device("cuda")
    sh = torch.tensor(shapes, dtype=torch.long)
    lsi = fda_oracle.level_start_index_of(sh)
    N = int(sh.prod(1).sum())
    step = HostStreamedStep((B, N, G, D), torch.bfloat16, (B, Q, G, 2 * K * 4), torch.float32, K, sh.to(dev), lsi.to(dev), dev,
                            chunk_queries=25)
    out_h = torch.empty(B, Q, G * D, dtype=torch.bfloat16).pin_memory()
    gv_h = torch.empty(B, N, G, D, dtype=torch.bfloat16).pin_memory()
    gp_h = torch.empty(B, Q, G, 2 * K * 4).pin_memory()
    for seed in (51, 52):
        value, _, _, packed, grad_out = fda_oracle.make_inputs(shapes, B, Q, G, D, K, seed=seed, lo=-0.2, hi=1.2)
        value_h, packed_h, go_h = value.bfloat16().pin_memory(), packed.pin_memory(), grad_out.bfloat16().pin_memory()
        assert capi.binning_applies(value_h.to(dev)[:1], packed_h.to(dev)[:1, :25], K)
        step.run(value_h, packed_h, go_h, out_h, gv_h, gp_h)
        torch.cuda.synchronize()
        ref_out, ref_gv, ref_gp = fda_oracle.fused_forward_backward(value_h, sh, packed_h, go_h, K)
        for got, ref in ((out_h, ref_out), (gv_h, ref_gv), (gp_h, ref_gp)):
            assert (got.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    assert step.h2d_bytes == value_h.numel() * 2 + packed_h.numel() * 4 + go_h.numel() * 2
    assert step.d2h_bytes == out_h.numel() * 2 + gv_h.numel() * 2 + gp_h.numel() * 4
