"""Error behaviour at the C-ABI boundary: violations the reference turns into host asserts come
back as status codes / Python exceptions, never as a device fault."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bad_arguments_raise():
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda as quant

    x = torch.zeros(256, 128, dtype=torch.bfloat16, device="cuda")
    ld = torch.zeros(128, 32, dtype=torch.bfloat16, device="cuda")
    sm = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        quant(x.float(), lora_down=ld, smooth=sm, fp4=True)          # wrong dtype
    with pytest.raises(ValueError):
        quant(x[:, :96], lora_down=ld, smooth=sm, fp4=True)           # not contiguous
    with pytest.raises(ValueError):
        quant(torch.zeros(256, 96, dtype=torch.bfloat16, device="cuda"), lora_down=ld[:96].contiguous(),
              smooth=sm[:96].contiguous(), fp4=True)                   # K not a multiple of 128
    with pytest.raises(ValueError):
        quant(x.cpu(), lora_down=ld, smooth=sm, fp4=True)             # no CPU path
    with pytest.raises(ValueError):
        # fuse_glu halves the channel count: a [256, 256] input is K = 128, which does not match smooth / lora_down
        quant(torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda"), lora_down=ld, smooth=sm, fp4=True, fuse_glu=True,
              output=torch.empty(256, 128, dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError):
        # an input narrower than the parameters is allowed (K_in), but only in steps of 8 columns
        quant(torch.zeros(256, 100, dtype=torch.bfloat16, device="cuda"), lora_down=ld, smooth=sm, fp4=True)
    # the context is still healthy
    out = quant(x, lora_down=ld, smooth=sm, fp4=True)
    torch.cuda.synchronize()
    assert int(out[0].sum()) == 0
