import torch

from innova_b200.models.multimodal import (AllModalityMoE, AudioEncoderConfig, AudioTransformer, ContrastiveAlignmentHead, FusionConfig,
                                            ImageNetClassifier, JointMultimodalModel, MelSpectrogram, ModalityEncoder, MultiModalTokenizer,
                                            OCRPipeline, Perceiver, SpeechRecognizer, VideoUnderstanding, ViTConfig, VisionTransformer)
from innova_b200.utils.tokenizer import ByteTokenizer

VIT = ViTConfig(image_size=32, patch_size=8, hidden=32, layers=1, heads=2, ffn=64)
AUD = AudioEncoderConfig(n_mels=16, hidden=32, layers=1, heads=2, ffn=64, max_frames=64)


def test_encoders_shapes_and_mel():
    torch.manual_seed(0)
    v = VisionTransformer(VIT)
    assert v(torch.randn(2, 3, 32, 32)).shape == (2, 17, 32)
    mel = MelSpectrogram(sample_rate=8000, n_fft=128, hop=64, n_mels=16)
    t = torch.arange(4000) / 8000.0
    lo, hi = mel(torch.sin(2 * torch.pi * 300 * t)[None]), mel(torch.sin(2 * torch.pi * 3000 * t)[None])
    assert lo.shape[-1] == 16 and lo[0].mean(0).argmax() < hi[0].mean(0).argmax()     # higher tone -> higher mel bin
    a = AudioTransformer(AUD)
    out = a(torch.randn(2, 3200))
    assert out.shape[0] == 2 and out.shape[2] == 32 and out.shape[1] <= 64
    assert Perceiver(hidden=32, latents=4, heads=2, ffn=64, layers=1)(torch.randn(2, 50, 32)).shape == (2, 4, 32)


def test_contrastive_head_learns_alignment():
    torch.manual_seed(1)
    a = torch.randn(8, 16)
    b = a @ torch.randn(16, 12) + 0.01 * torch.randn(8, 12)
    head = ContrastiveAlignmentHead(16, 12, d_joint=8)
    opt = torch.optim.Adam(head.parameters(), lr=5e-2)
    first = None
    for _ in range(150):
        loss, logits = head(a, b)
        first = first or float(loss)
        opt.zero_grad(); loss.backward(); opt.step()
    assert float(loss) < 0.3 * first and bool((logits.argmax(-1) == torch.arange(8)).all())


def test_joint_model_uses_the_image_and_trains():
    torch.manual_seed(2)
    m = JointMultimodalModel(vocab=20, hidden=32, vit=VIT, audio=AUD, fusion=FusionConfig(hidden=32, heads=2, ffn=64, layers=1), max_len=16)
    imgs = torch.stack([torch.full((3, 32, 32), -1.0), torch.full((3, 32, 32), 1.0)])
    ids = torch.tensor([[1, 2, 3, 4], [1, 2, 3, 4]])
    labels = torch.tensor([[5, 5, 5, 5], [9, 9, 9, 9]])                   # only the image tells the two apart
    opt = torch.optim.Adam(m.parameters(), lr=1e-2)
    for _ in range(80):
        loss = torch.nn.functional.cross_entropy(m(ids, image=imgs).flatten(0, 1), labels.flatten())
        opt.zero_grad(); loss.backward(); opt.step()
    assert float(loss) < 0.2
    pred = m(ids, image=imgs).argmax(-1)
    assert pred[0, -1] == 5 and pred[1, -1] == 9
    assert m.generate(ids[:1], 3, image=imgs[:1]).shape == (1, 7)
    assert m(ids, audio=torch.randn(2, 3200)).shape == (2, 4, 20)        # any subset of modalities


def test_task_heads_and_moe():
    torch.manual_seed(3)
    assert ImageNetClassifier(10, VIT)(torch.randn(2, 3, 32, 32)).shape == (2, 10)
    assert VideoUnderstanding(5, VIT, temporal_layers=1)(torch.randn(2, 3, 3, 32, 32)).shape == (2, 5)
    asr = SpeechRecognizer(12, AUD)
    wav = torch.randn(2, 3200)
    loss = asr.loss(wav, torch.tensor([[1, 2, 3], [4, 5, 6]]), torch.tensor([3, 3]))
    assert torch.isfinite(loss) and len(asr.transcribe(wav)) == 2
    ocr = OCRPipeline(12, VIT)
    assert ocr(torch.randn(2, 3, 32, 32)).shape == (2, 16, 13)
    moe = AllModalityMoE(hidden=32, ffn=48, experts=4, top_k=2)
    x = torch.randn(2, 6, 32)
    y, aux = moe(x, "audio")
    assert y.shape == x.shape and float(aux) >= 1.0 - 1e-4 and not torch.equal(moe(x, "vision")[0], y)
    enc = ModalityEncoder(50, hidden=32, layers=1, heads=2, ffn=64)
    assert enc(torch.randint(0, 50, (2, 7))).shape == (2, 7, 32)
    tok = MultiModalTokenizer(ByteTokenizer())
    ids = tok.encode("hi", ["image"])
    assert ids[:2] == [256, 257] and tok.decode(ids) == "hi" and tok.vocab_size == 262
