"""Per-epoch crop / flip augmentation: draws, geometry, trainer hook."""
import torch


def test_crop_flip_geometry_and_determinism():
    from noeira_b200.training.augment import CropFlipAugmenter, crop_flip_draws
    x = torch.arange(3 * 2 * 8 * 8, dtype=torch.float32).reshape(3, 2, 8, 8) + 1
    aug = CropFlipAugmenter(pad=2)
    a, b = torch.empty_like(x), torch.empty_like(x)
    aug.augment(a, x, epoch=3, seed=7)
    aug.augment(b, x, epoch=3, seed=7)
    assert torch.equal(a, b)                                   # a function of (seed, epoch, index) only
    aug.augment(b, x, epoch=4, seed=7)
    assert not torch.equal(a, b)
    dx, dy, flip = crop_flip_draws(3, 3, 7, 2, "cpu")
    for n in range(3):
        ref = torch.nn.functional.pad(x[n], (2, 2, 2, 2))[:, dy[n]: dy[n] + 8, dx[n]: dx[n] + 8]
        if flip[n]:
            ref = ref.flip(-1)
        assert torch.equal(a[n], ref)
    # NHWC gives the same pictures
    nh = CropFlipAugmenter(pad=2, layout="nhwc")
    c = torch.empty(3, 8, 8, 2)
    nh.augment(c, x.permute(0, 2, 3, 1).contiguous(), epoch=3, seed=7)
    assert torch.equal(c.permute(0, 3, 1, 2), a)
    # draws cover the whole range
    dx, dy, flip = crop_flip_draws(4096, 0, 1, 4, "cpu")
    assert set(dx.tolist()) == set(range(9)) and set(dy.tolist()) == set(range(9)) and 0.4 < flip.float().mean() < 0.6


def test_trainer_refills_the_buffer_each_epoch():
    from noeira_b200 import nn
    from noeira_b200.training.augment import CropFlipAugmenter, IdentityAugmenter
    from noeira_b200.training.trainer import Trainer
    nn.manual_seed(0)
    x = torch.randn(64, 1, 6, 6)
    y = torch.randint(0, 3, (64,))

    class Flat(nn.Module):
        def forward(self, x):
            self._s = x.shape
            return x.reshape(x.shape[0], -1)

        def vjp(self, dy):
            return dy.reshape(self._s)

    model = nn.Sequential(Flat(), nn.LinearReLU(36, 16, need_input_grad=False), nn.Linear(16, 3, out_fp32=True))
    tr = Trainer(model, x, y, batch=16, lr=1e-2, augmenter=CropFlipAugmenter(pad=1), seed=5)
    assert tr.x.data_ptr() != x.data_ptr() and torch.equal(tr.raw_x, x)
    e0 = tr.x.clone()
    tr.train_epoch(1)
    e1 = tr.x.clone()
    assert not torch.equal(e0, e1)                             # epoch 1 drew other crops into the same buffer
    tr2 = Trainer(model, x, y, batch=16, augmenter=IdentityAugmenter())
    assert tr2.x.data_ptr() == x.data_ptr()                    # a no-op augmenter costs no buffer
