"""Crop / flip augmentation kernel against the tensor-program oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kernel_matches_reference(layout, dtype):
    from noeira_b200.training.augment import CropFlipAugmenter
    torch.manual_seed(0)
    shape = (37, 3, 32, 32) if layout == "nchw" else (37, 32, 32, 3)
    x = torch.randn(*shape, device="cuda").to(dtype)
    aug = CropFlipAugmenter(pad=4, layout=layout)
    out = torch.empty_like(x)
    aug.augment(out, x, epoch=5, seed=11)
    torch.cuda.synchronize()
    assert torch.equal(out, aug.reference(x, 5, 11))
