"""Text-to-image diffusion sampler and Griffin-Lim synthesis (CPU)."""
import math

import torch

from innova_b200.models.generative import AudioSynthesizer, DiffusionUNet, TextToImage
from innova_b200.models.multimodal import MelSpectrogram


def test_text_to_image_smooth_proxy_is_deterministic_and_bounded():
    m = TextToImage(latent_dim=16, image_size=64, predictor="smooth")
    a = m.generate("a red square", steps=20)
    b = m.generate("a red square", steps=20)
    c = m.generate("a blue circle", steps=20)
    assert a.shape == (3, 64, 64) and torch.equal(a, b)
    assert a.abs().max() <= 1.0 and torch.isfinite(a).all()
    assert not torch.equal(a, c)                      # the prompt conditions the sample


def test_smooth_eps_matches_the_neighbour_loop():
    x = torch.randn(1, 2, 5, 4)
    got = TextToImage._smooth_eps(x)
    ref = torch.zeros_like(x)
    H, W = 5, 4
    for c in range(2):
        for i in range(H):
            for j in range(W):
                vals = [x[0, c, i, j]]
                if i > 0: vals.append(x[0, c, i - 1, j])
                if i < H - 1: vals.append(x[0, c, i + 1, j])
                if j > 0: vals.append(x[0, c, i, j - 1])
                if j < W - 1: vals.append(x[0, c, i, j + 1])
                ref[0, c, i, j] = (x[0, c, i, j] - sum(vals) / len(vals)) * 0.5
    assert torch.allclose(got, ref, atol=1e-6)


def test_unet_training_reduces_noise_prediction_error():
    torch.manual_seed(0)
    m = TextToImage(latent_dim=16, image_size=64, train_steps=100)
    imgs = torch.stack([torch.full((3, 64, 64), 0.8), torch.full((3, 64, 64), -0.8)])
    prompts = ["bright", "dark"]
    opt = torch.optim.Adam(m.parameters(), lr=2e-3)
    first = None
    for it in range(40):
        torch.manual_seed(it % 4)                     # a few fixed (t, noise) draws: the loss is comparable across steps
        loss = m.training_loss(imgs, prompts, drop_prompt=0.0)
        opt.zero_grad(); loss.backward(); opt.step()
        first = first if first is not None else float(loss.detach())
    assert float(loss) < 0.5 * first
    out = m.generate(prompts, steps=10)
    assert out.shape == (2, 3, 64, 64) and torch.isfinite(out).all()


def test_unet_shapes_odd_resolution():
    u = DiffusionUNet(3, (16, 32), cond_dim=8)
    y = u(torch.randn(2, 3, 9, 9), torch.tensor([3, 50]), torch.randn(2, 8))
    assert y.shape == (2, 3, 9, 9)


def test_griffin_lim_recovers_a_tone():
    sr, n_fft, hop = 16000, 512, 128
    t = torch.arange(sr // 2) / sr
    wav = 0.5 * torch.sin(2 * math.pi * 440.0 * t)
    mel = MelSpectrogram(sr, n_fft, hop, n_mels=64)(wav[None])[0].T          # [n_mels, frames], log of power
    syn = AudioSynthesizer(sr, n_fft, hop, n_mels=64, iters=16, power=2.0)
    out = syn.synthesize(mel)
    assert out.dim() == 1 and abs(out.numel() - wav.numel()) <= n_fft
    spec = torch.fft.rfft(out * torch.hann_window(out.numel())).abs()
    peak_hz = float(spec.argmax()) * sr / out.numel()
    assert abs(peak_hz - 440.0) < 40.0
    # more rounds of phase estimation realise the magnitudes better than the random start
    rough = AudioSynthesizer(sr, n_fft, hop, n_mels=64, iters=1, power=2.0)
    assert syn.spectral_convergence(out, mel) < rough.spectral_convergence(rough.synthesize(mel), mel)
    assert syn.synthesize(torch.zeros(0)).numel() == 0
    assert syn.synthesize(torch.stack([mel, mel])).shape[0] == 2
