"""nunchaku_b200.weights (the shipped packers / SVDQuant-lite quantiser) against the reference
packer's golden vectors and the oracle's independently written layouts."""
import numpy as np
import torch

from nunchaku_b200 import weights as W
from oracle import fmt
from oracle import layouts as L
from oracle import svdq_ref as R


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def test_packers_match_reference_golden(golden):
    codes = (torch.from_numpy(golden["wgt_codes_in"]).to(torch.int32) & 0xF).to(torch.uint8)
    assert np.array_equal(W.pack_weight_codes(codes).view(torch.uint8).numpy(), golden["wgt_codes_packed"])
    v = _bf16(golden["vector_in"])
    assert np.array_equal(W.pack_vector(v).view(torch.int16).numpy(), golden["vector_packed"])
    ws = _bf16(golden["wscales_in"]).t().contiguous()
    assert np.array_equal(W.pack_int4_wscales(ws).view(torch.int16).numpy(), golden["wscales_packed"])
    ms = torch.from_numpy(golden["wmscales_in"]).t().contiguous().view(torch.float8_e4m3fn)
    assert np.array_equal(W.pack_nvfp4_wscales(ms).view(torch.uint8).numpy(), golden["wmscales_packed"])
    assert np.array_equal(W.pack_lora_up(_bf16(golden["lora_up_in"])).view(torch.int16).numpy(), golden["lora_up_packed"])
    assert np.array_equal(W.pack_lora_down(_bf16(golden["lora_down_in"])).view(torch.int16).numpy(), golden["lora_down_packed"])


def test_code_encoders_match_oracle():
    v = torch.cat([torch.randn(4096) * 3, torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.0, -0.1, 9.0])])
    assert torch.equal(W.e2m1_codes(v), fmt.e2m1_encode(v))
    assert torch.equal(W.int4_codes(v), fmt.int4_encode(v, False))


def test_svdquant_state_dict_reconstructs_weight():
    torch.manual_seed(0)
    for precision in ("nvfp4", "int4"):
        lin = torch.nn.Linear(256, 384, dtype=torch.bfloat16)
        xa = torch.rand(256) * 4 + 0.5
        sd = W.svdquant_state_dict(lin.weight, lin.bias, xa, rank=32, precision=precision)
        fp4 = precision == "nvfp4"
        smooth = L.ref_unpack_vector(sd["smooth_factor"])
        wcodes = L.ref_unpack_wgt_codes(sd["qweight"], 256)
        if fp4:
            ws = L.ref_unpack_wmscales(sd["wscales"].view(torch.uint8))
        else:
            ws = L.ref_unpack_wscales(sd["wscales"])
        o = R.Linear(256, 384, 32, fp4, wcodes, ws, smooth, L.ref_unpack_lora_down(sd["proj_down"]),
                     L.ref_unpack_lora_up(sd["proj_up"]), L.ref_unpack_vector(sd["bias"]),
                     float(sd["wtscale"].item()) if fp4 else 1.0, L.ref_unpack_vector(sd["wcscales"]) if fp4 else None)
        # effective weight seen by an un-smoothed activation: (W_q + up @ down_smoothed) / smooth
        eff = o.dequant_weight() / smooth.float()[None, :] + o.lora_up.float() @ o.lora_down.float()
        assert R.rel_l2(eff, lin.weight.float()) < 0.12
