"""The init-then-use facades: containers round-trip through PGM / PPM files, every engine refuses use before init and
produces the documented shapes after."""
import os

import pytest
import torch

from innova_b200.models.modalities import api


def test_image_and_video_containers(tmp_path):
    img = api.Image(6, 4, 3)
    assert (img.width, img.height, img.channels, img.numel()) == (6, 4, 3, 72)
    img.pixels = torch.rand(4, 6, 3)
    p = str(tmp_path / "a.ppm")
    img.save(p)
    back = api.Image.load(p)
    assert (back.width, back.height, back.channels) == (6, 4, 3) and (back.pixels - img.pixels).abs().max() <= 0.5 / 255 + 1e-6
    assert back.to_tensor().shape == (3, 4, 6) and torch.equal(api.Image.from_tensor(back.to_tensor()).pixels, back.pixels)
    with open(tmp_path / "c.pgm", "wb") as f:
        f.write(b"P5\n# a comment\n3 2\n65535\n" + bytes([0, 0, 255, 255, 128, 0, 0, 1, 0, 2, 0, 3]))
    grey = api.Image.load(str(tmp_path / "c.pgm"))
    assert grey.channels == 1 and grey.pixels[0, :, 0].tolist() == pytest.approx([0.0, 1.0, 32768 / 65535])
    for bad in (b"P3\n1 1\n255\n0 0 0", b"P6\n2 2\n255\n\x00\x00"):
        (tmp_path / "bad.ppm").write_bytes(bad)
        with pytest.raises(ValueError):
            api.Image.load(str(tmp_path / "bad.ppm"))
    with pytest.raises(ValueError):
        api.Image(2, 2, 2).save(str(tmp_path / "x.ppm"))
    d = tmp_path / "clip"
    d.mkdir()
    for i in range(3):
        fr = api.Image(8, 8, 1)
        fr.pixels = torch.full((8, 8, 1), i / 4)
        fr.save(str(d / f"f{i:02d}.pgm"))
    (d / "notes.txt").write_text("ignored")
    vid = api.Video.load(str(d), fps=12.0)
    assert vid.num_frames() == 3 and (vid.width, vid.height) == (8, 8) and vid.fps() == 12.0 and vid.to_tensor().shape == (3, 8, 8)
    assert float(vid.frame(2).pixels.mean()) == pytest.approx(0.5, abs=1 / 255) and api.Video().to_tensor().numel() == 0
    odd = api.Image(4, 4, 1)
    odd.save(str(d / "f99.pgm"))
    with pytest.raises(ValueError):
        api.Video.load(str(d))


def test_engines_refuse_use_before_init_and_work_after():
    for eng, arg in ((api.AudioEncoder(), [0.0] * 800), (api.MelSpectrogram(), [0.0] * 800), (api.AudioFeatureExtractor(), [0.0] * 800),
                     (api.VisionEncoder(), torch.rand(3, 8, 8)), (api.VideoEncoder(), torch.rand(4, 8, 8)), (api.OCREngine(), torch.rand(32, 128)),
                     (api.TextEncoder(), "hi")):
        assert not eng.is_initialized()
        with pytest.raises(RuntimeError):
            (eng.encode if hasattr(eng, "encode") else eng.extract if hasattr(eng, "extract") else eng.recognize)(arg)
    with pytest.raises(RuntimeError):
        api.ImageClassifier().classify(torch.rand(3, 8, 8))
    torch.manual_seed(0)
    pcm = torch.randn(4000).tolist()
    mel = api.MelSpectrogram()
    mel.init(api.MelSpectrogram.Config(n_mels=20))
    m = mel.extract(pcm)
    assert m.shape == (20, mel.feature_length(4000)) == (20, 23) and abs(float(m.mean())) < 1e-4 and float(m.std()) == pytest.approx(1.0, abs=1e-3)
    fx = api.AudioFeatureExtractor()
    fx.init(16000, 20, n_encoder_layers=1, d_model=32, n_heads=4)
    feats = fx.extract(pcm)
    assert feats.n_frames == 23 and feats.encoder_output.shape == (23, 32) and feats.sample_rate == 16000 and fx.encoder.d_model == 32
    vis = api.VisionEncoder()
    assert vis.hidden_size == 0
    vis.init(api.VisionEncoder.Config(img_size=32, patch_size=8, hidden_size=32, num_layers=1, num_heads=4), num_classes=5)
    assert vis.hidden_size == 32 and vis.encode(torch.rand(3, 32, 32)).shape == (1, 17, 32) and vis.encode(torch.rand(1, 50, 40)).shape == (1, 17, 32)
    img = api.Image(20, 10, 3)
    img.pixels = torch.rand(10, 20, 3)
    assert vis.encode(img).shape == (1, 17, 32)
    clf = api.ImageClassifier()
    clf.init(vis.config, num_classes=5)
    r = clf.classify(img)
    assert 0 <= r.top_class < 5 and len(r.logits) == 5 and 0.2 <= r.top_confidence <= 1 and r.top_class == max(range(5), key=r.logits.__getitem__)
    ve = api.VideoEncoder()
    ve.init(api.VideoEncoder.Config(tube_size=2, patch_size=8, hidden_size=32, num_layers=1, num_heads=4, max_frames=12))
    assert ve.encode(torch.rand(20, 16, 16)).shape == (2, 32) and ve.encode([torch.rand(16, 16)] * 4).shape == (1, 32)
    ocr = api.OCREngine()
    ocr.init(api.OCREngine.Config(hidden_size=32, num_layers=1, num_heads=4))
    res = ocr.recognize(torch.rand(48, 160))
    assert isinstance(res.full_text, str) and all(0 <= b.x0 < b.x1 <= 1 and 0 <= b.y0 < b.y1 <= 1 and 0 < b.confidence <= 1 for b in res.boxes)
    assert [(b.y0, b.x0) for b in res.boxes] == sorted((b.y0, b.x0) for b in res.boxes) and ocr.recognize(torch.rand(8, 8)).boxes == []
    te = api.TextEncoder()
    te.init(api.TextEncoder.Config(vocab_size=300, max_seq_len=16, hidden_size=32, num_layers=1, num_heads=4))
    assert te.encode("héllo").shape == (6, 32) and te.encode([1, 2, 3]).shape == (3, 32) and te.encode("").shape == (1, 32)
    assert api.TextDecoder.decode([104, 105, 999]) == "hi" and api.TextDecoder.decode(torch.eye(256)[[111, 107]]) == "ok"
