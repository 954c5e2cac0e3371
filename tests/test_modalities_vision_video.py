"""Image, vision and video modalities: helper ops against naive loops, shapes of every head, determinism of the sampler, and a
short training run that shows gradients reach the encoders."""
import math

import pytest
import torch
import torch.nn.functional as F

from innova_b200.models.modalities import image as I, video as VD, vision as V
from innova_b200.models.modalities._blocks import patchify, sinusoid_table, unpatchify


def test_patchify_layout_sinusoids_and_schedule():
    img = torch.arange(2 * 3 * 4 * 6, dtype=torch.float32).view(2, 3, 4, 6)
    p = patchify(img, 2)
    assert p.shape == (2, 6, 12)
    # patch (row 1, col 2), channel 1, pixel (1, 0)
    assert p[1, 1 * 3 + 2, 1 * 4 + 1 * 2 + 0] == img[1, 1, 1 * 2 + 1, 2 * 2 + 0]
    assert torch.equal(unpatchify(p, 2, 3, 4, 6), img) and patchify(torch.zeros(1, 1, 5, 7), 2).shape == (1, 6, 4)
    t = sinusoid_table(5, 7)
    assert t.shape == (5, 7) and (t[:, 6] == 0).all()
    assert float(t[3, 2]) == pytest.approx(math.sin(3 / 10000 ** (2 / 7)), abs=1e-6) and float(t[3, 3]) == pytest.approx(math.cos(3 / 10000 ** (2 / 7)), abs=1e-6)
    s = I.cosine_schedule(10)
    assert s.shape == (10, 3) and torch.allclose(s[:, 1] + s[:, 2], torch.ones(10)) and (s[1:, 0] <= s[:-1, 0]).all()
    assert float(s[0, 0]) == pytest.approx(math.cos((0.1 + 0.008) / 1.008 * math.pi / 2) ** 2, rel=1e-5) and float(s[-1, 0]) == pytest.approx(1e-3)
    assert torch.allclose(torch.cumprod(s[:5, 1], 0), s[:5, 0], rtol=1e-5)
    assert I.patch_size_for(64) == 8 and I.patch_size_for(30) == 3 and I.patch_size_for(16) == 4


def test_conv_helpers_match_naive_definitions():
    torch.manual_seed(0)
    x = torch.randn(2, 3, 6, 5)
    cols = I.im2col(x, 3, 3, 1, 1, 1, 1)
    assert cols.shape == (2 * 6 * 5, 27)
    xp = F.pad(x, (1, 1, 1, 1))
    assert torch.allclose(cols[(1 * 6 + 2) * 5 + 3], xp[1, :, 2:5, 3:6].reshape(-1))
    w = torch.randn(4, 27)
    conv = (cols @ w.T).view(2, 6, 5, 4).permute(0, 3, 1, 2)
    block = I.ConvBlock(3, 4, 3, 1, 1)
    with torch.no_grad():
        block.conv_weight.copy_(w)
    assert torch.allclose(block(x), conv, atol=1e-5)
    mean, var, bias = torch.randn(4), torch.rand(4) + 0.5, torch.randn(4)
    bn = I.conv2d_batch_norm(x, w, bias, mean, var)
    assert torch.allclose(bn, (conv - mean.view(1, 4, 1, 1)) / torch.sqrt(var.view(1, 4, 1, 1) + 1e-5) + bias.view(1, 4, 1, 1), atol=1e-4)
    assert I.max_pool2d(x, 2, 2).shape == (2, 3, 3, 2) and float(I.max_pool2d(x, 2, 2)[0, 0, 0, 0]) == float(x[0, 0, :2, :2].max())
    assert torch.allclose(I.global_avg_pool2d(x), x.mean((2, 3))) and I.adaptive_avg_pool2d(x, 3, 1).shape == (2, 3, 3, 1)
    up = I.adaptive_avg_pool2d(torch.arange(4.0).view(1, 1, 2, 2), 4, 4)
    assert up[0, 0].tolist() == [[0, 0, 1, 1], [0, 0, 1, 1], [2, 2, 3, 3], [2, 2, 3, 3]]
    r = I.ResidualBlock(3)
    assert r(x).shape == x.shape and (r(x) >= 0).all()
    assert I.ConvBlock(3, 8, 7, 2, 3)(torch.randn(1, 3, 32, 32)).shape == (1, 8, 16, 16)


def test_image_encoder_decoder_generator():
    torch.manual_seed(0)
    gen = I.ImageGenerator(img_size=32, hidden_size=32, num_layers=1, num_heads=4, latent_dim=8)
    img = torch.rand(2, 3, 32, 32)
    feats = gen.encoder.encode(img)
    assert feats.shape == (2, 64, 32) and gen.encoder.project_to_latent(feats).shape == (2, 8)
    assert gen.encoder.extract_features(img, True).shape == (2, 1, 32) and gen.encoder.extract_multi_scale_features(img).shape == (2, 1, 32)
    assert gen.decoder.decode(torch.randn(2, 8)).shape == (2, 3, 32, 32) and gen.decoder.decode_v2(torch.randn(2, 8), 2).shape == (2, 3, 32, 32)
    assert gen.decoder.upscale(feats).shape == (2, 64, 64) and gen.noise_schedule.shape == (1000, 3)
    a = gen.generate(img, 3, generator=torch.Generator().manual_seed(5))
    b = gen.generate(img, 3, generator=torch.Generator().manual_seed(5))
    c = gen.generate(torch.randn(2, 8), 3, generator=torch.Generator().manual_seed(6))
    assert torch.equal(a.generated, b.generated) and a.generated.shape == (2, 3, 32, 32) and not torch.equal(a.latents, c.latents)
    assert len(a.scores) == 2 and all(0 < s <= 1 for s in a.scores)
    assert a.scores[0] == pytest.approx(1 / (1 + float(a.latents[0].var(unbiased=False))), rel=1e-4)
    # one denoising step follows the ancestral update
    x, cond = torch.randn(2, 8), torch.randn(2, 8)
    eps = gen.predict_noise(x, cond, 1)
    assert eps.shape == (2, 8)
    # an auto-encoding objective trains through encoder and decoder
    opt = torch.optim.Adam(list(gen.encoder.parameters()) + list(gen.decoder.parameters()), 2e-3)
    losses = []
    for _ in range(20):
        rec = gen.decoder.decode(gen.encoder.project_to_latent(gen.encoder.encode(img)))
        loss = F.mse_loss(rec, img)
        losses.append(float(loss.detach()))
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert losses[-1] < losses[0]


def test_vision_encoder_heads_and_preprocessing():
    torch.manual_seed(0)
    m = V.VisionEncoder(img_size=32, patch_size=8, hidden_size=32, num_layers=2, num_heads=4, num_classes=7, max_detections=20, caption_vocab=30)
    assert torch.allclose(m.pos_embed[0], sinusoid_table(17, 32))
    x = torch.rand(2, 3, 32, 32)
    enc = m.encode(x)
    assert enc.shape == (2, 17, 32) and m.classify(enc).shape == (2, 7)
    boxes = m.detect_objects(enc)
    assert boxes.shape == (2, 20, 4) and (boxes[:, 16:] == 0).all()
    order = m.class_head(enc[:, 1:]).amax(-1).argsort(1, descending=True)
    assert torch.allclose(boxes[0, 0], m.bbox_head(enc[0, 1 + order[0, 0]])) and torch.allclose(boxes[1, 15], m.bbox_head(enc[1, 1 + order[1, 15]]))
    cap = m.generate_caption(enc, 4)
    assert cap.shape == (2, 4, 30)
    ctx = m.caption_proj(enc[:, 0])
    assert torch.allclose(cap[:, 0], (m.caption_embed[1] + ctx) @ m.caption_embed.T, atol=1e-5)
    nxt = cap[:, 0].argmax(-1)
    assert torch.allclose(cap[:, 1], (m.caption_embed[nxt] + ctx) @ m.caption_embed.T, atol=1e-5)
    res = m(x, V.VisionTask.DETECT)
    assert res.bboxes is not None and res.class_logits.shape == (2, 7) and 0 < res.confidence <= 1
    assert m(x, V.VisionTask.CAPTION).captions.shape == (2, 17, 30) and m(x, V.VisionTask.CLASSIFY).bboxes is None
    assert m.encode(torch.rand(1, 3, 48, 40)).shape == (1, 1 + 6 * 5, 32)                 # interpolated positions
    pe = m.interpolate_pos_encoding(4, 4)
    assert torch.allclose(pe, m.pos_embed) and m.interpolate_pos_encoding(8, 8).shape == (1, 65, 32)
    assert m.encode_multiscale([x, torch.rand(2, 3, 16, 16)]).shape == (2, 34, 32) and m.encode_multiscale([]).shape == (1, 1, 32)
    maps = m.extract_attention_maps(x)
    assert len(maps) == 2 and maps[0].shape == (2, 17, 17) and torch.allclose(maps[1].sum(-1), torch.ones(2, 17), atol=1e-5)
    assert m.compute_self_attention(enc, enc).shape == (2, 17, 2, 17)
    assert V.Conv2dPatchEmbed(3, 16, 8)(x).shape == (2, 16, 16)
    ln = V.LayerNorm2D(24)
    y = ln(enc)
    assert y.shape == (2, 17, 24) and torch.allclose(y.mean(-1), torch.zeros(2, 17), atol=1e-5)
    fx = V.ViTFeatureExtractor(32, 8)
    assert fx.extract_patches(x).shape == (2, 16, 192)
    n = fx.normalize(x)
    assert float(n[0, 1, 3, 4]) == pytest.approx((float(x[0, 1, 3, 4]) - 0.456) / 0.224, rel=1e-5)
    assert torch.allclose(fx.normalize_quantized(x), n, atol=1e-4)
    r = fx.resize(x, 48, 16)
    ih, iw = 5 * 32 / 48, 3 * 32 / 16
    i0, j0 = int(ih), int(iw)
    dh, dw = ih - i0, iw - j0
    want = ((x[0, 0, i0, j0] * (1 - dw) + x[0, 0, i0, j0 + 1] * dw) * (1 - dh) + (x[0, 0, i0 + 1, j0] * (1 - dw) + x[0, 0, i0 + 1, j0 + 1] * dw) * dh)
    assert r.shape == (2, 3, 48, 16) and float(r[0, 0, 5, 3]) == pytest.approx(float(want), rel=1e-5) and torch.equal(fx.resize(x, 32, 32), x)
    assert torch.equal(fx.center_crop(x, 16), x[:, :, 8:24, 8:24])
    er = fx.random_erasing(x, 1.0, 0.25, generator=torch.Generator().manual_seed(0))
    changed = (er != x).any(1)
    assert changed[0].any() and 0.05 < changed[0].float().mean() < 0.6 and torch.equal(fx.random_erasing(x, 0.0, 0.25), x)
    rows = changed[0].any(1).nonzero().flatten()
    assert float(er[0, 2, rows[0], changed[0][rows[0]].nonzero()[0, 0]]) == pytest.approx(float(x[0, 2].mean()), rel=1e-5)


def _naive_flow(prev, curr, bs, sr):
    B, H, W = prev.shape
    f = torch.zeros(B, H, W, 2)
    for b in range(B):
        for i in range(0, H - bs + 1, bs // 2):
            for j in range(0, W - bs + 1, bs // 2):
                best, bdy, bdx = 1e30, 0, 0
                for dy in range(max(0, i - sr), min(H - bs, i + sr) + 1):
                    for dx in range(max(0, j - sr), min(W - bs, j + sr) + 1):
                        sad = float((prev[b, i:i + bs, j:j + bs] - curr[b, dy:dy + bs, dx:dx + bs]).abs().sum())
                        if sad < best:
                            best, bdy, bdx = sad, dy - i, dx - j
                f[b, i:i + bs, j:j + bs, 0] = bdx
                f[b, i:i + bs, j:j + bs, 1] = bdy
    return f


def test_video_ops_flow_and_encoder():
    torch.manual_seed(0)
    prev = torch.rand(2, 20, 28)
    curr = torch.roll(prev, shifts=(1, -2), dims=(1, 2))
    flow = VD.compute_optical_flow(prev, curr, 8, 3)
    assert torch.equal(flow, _naive_flow(prev, curr, 8, 3))
    assert flow[0, 8:12, 8:12, 0].unique().tolist() == [-2.0] and flow[0, 8:12, 8:12, 1].unique().tolist() == [1.0]
    assert (VD.compute_optical_flow(prev[:, :4], curr[:, :4], 8, 3) == 0).all()
    x = torch.randn(1, 2, 5, 6, 7)
    w, b = torch.randn(3, 2, 2, 3, 3), torch.randn(3)
    y = VD.conv3d_forward(x, w, b, 1, 2, 2)
    assert y.shape == (1, 3, 4, 2, 3)
    assert float(y[0, 1, 2, 1, 2]) == pytest.approx(float((x[0, :, 2:4, 2:5, 4:7] * w[1]).sum() + b[1]), rel=1e-4)
    assert VD.max_pool3d(x, 2, 2, 2, 2, 2, 2).shape == (1, 2, 2, 3, 3)
    f = torch.randn(2, 5, 4)
    assert torch.allclose(VD.temporal_pooling(f, "mean"), f.mean(1)) and torch.allclose(VD.temporal_pooling(f, "max"), f.amax(1))
    att = torch.softmax(f.mean(-1), 1)
    assert torch.allclose(VD.temporal_pooling(f, "attention"), (att[..., None] * f).sum(1), atol=1e-6) and (VD.temporal_pooling(f, "x") == 0).all()
    inc = VD.InceptionModule(3, 8)
    assert inc(torch.randn(2, 3, 10, 12)).shape == (2, 32, 10, 12)
    cfg = VD.VideoConfig(tube_depth=2, tube_height=8, tube_width=8, hidden_size=32, num_heads=4, head_dim=8, num_layers=1, clip_len=4, ffn_hidden=64, max_frames=16)
    enc = VD.SplitVideoEncoder(cfg)
    video = torch.rand(10, 24, 24)
    tubes = enc.extract_3d_tubes(video[:4])
    assert tubes.shape == (3 * 5 * 5, 128) and torch.equal(tubes[1 * 25 + 2 * 5 + 3], video[1:3, 8:16, 12:20].reshape(-1))
    assert enc.extract_3d_tubes(video[:1]).shape == (0, 128) and enc.encode_clip(video[:1]).shape == (1, 32)
    out = enc.encode(video)
    assert out.shape == (3, 32) and enc.encode_with_motion(video).shape == (3, 32) and enc.encode(video[:0]).shape == (1, 32)
    assert torch.allclose(enc.temporal_aggregate(out, "mean"), out.mean(0, keepdim=True)) and torch.equal(enc.temporal_aggregate(out, "last"), out[-1:])
    assert torch.equal(enc.temporal_aggregate(out, "first"), out[:1]) and enc.recognize_action(video) in enc.ACTIONS
    tt = VD.TemporalTransformer(cfg)
    assert tt([torch.randn(5, 32), torch.randn(32)]).shape == (2, 32) and tt([]).shape == (1, 32)
    bright = torch.zeros(2, 48, 48)
    bright[0, 16:32, 24:40] = 1.0
    assert enc.track_objects(bright) == [(24, 16), (24, 24)]
    mfe = VD.MotionFeatureExtractor(8, 2, 16)
    assert mfe.extract_motion(video[:3]).shape == (1, 16) and (mfe.extract_motion(video[:1]) == 0).all()
    still = video[:1].expand(3, -1, -1)
    assert (mfe.extract_motion(still) == 0).all()                  # no motion between identical frames
