"""CPU checks of the model, trainer and flat optimizer engine (PyTorch path, fp32)."""
import torch

from innova_b200.models import DenseModel, TransformerConfig, gpt2_small
from innova_b200.training.flat_engine import FlatParamEngine
from innova_b200.training.trainer import Trainer, TrainConfig
from innova_b200.utils.data import zipf_tokens, TokenLoader


def test_zipf_is_seeded_and_skewed():
    a = zipf_tokens(20000, 256, 1.1, seed=0)
    b = zipf_tokens(20000, 256, 1.1, seed=0)
    assert torch.equal(a, b)
    counts = torch.bincount(a, minlength=256)
    assert counts[0] > counts[10] > counts[200]
    assert int(a.max()) < 256 and int(a.min()) >= 0


def test_gpt2_style_cpu_training_reduces_loss():
    torch.manual_seed(0)
    cfg = gpt2_small(num_layers=2, hidden_size=64, num_heads=2, head_dim=32, ffn_hidden_size=128, vocab_size=256, max_seq_len=32, vocab_pad_to=1)
    model = DenseModel(cfg, dtype=torch.float32)
    tr = Trainer(model, TrainConfig(lr=3e-3, weight_decay=0.1))
    toks = zipf_tokens(8 * 32 + 1, 256, 1.1, seed=0)
    ids, labels = toks[:-1].view(8, 32), toks[1:].view(8, 32)
    first = float(tr.train_step(ids, labels))
    for _ in range(30):
        last = float(tr.train_step(ids, labels))
    assert last < first - 0.3


def test_llama_style_cpu_forward_and_reference_names():
    cfg = TransformerConfig(vocab_size=100, hidden_size=64, num_layers=2, num_heads=4, head_dim=16, ffn_hidden_size=96, num_kv_heads=2,
                            max_seq_len=16, vocab_pad_to=1)
    model = DenseModel(cfg, dtype=torch.float32)
    ids = torch.randint(0, 100, (2, 16))
    logits = model(ids)
    assert logits.shape == (2, 16, 100)
    sd = model.state_dict_reference()
    assert "layers.0.attention.q_proj.weight" in sd and "layers.1.ffn.gate_proj.weight" in sd and "lm_head.weight" in sd
    other = DenseModel(cfg, dtype=torch.float32, seed=7)
    other.load_reference_state(sd)
    assert torch.allclose(other(ids), logits, atol=1e-5)


def test_flat_engine_matches_torch_adamw():
    torch.manual_seed(1)
    lin = torch.nn.Linear(24, 40)
    ref = torch.nn.Linear(24, 40)
    ref.load_state_dict(lin.state_dict())
    eng = FlatParamEngine(lin, lr=1e-2, weight_decay=0.1, max_grad_norm=0.0)
    opt = torch.optim.AdamW([{"params": [ref.weight], "weight_decay": 0.1}, {"params": [ref.bias], "weight_decay": 0.0}], lr=1e-2)
    for _ in range(4):
        gw, gb = torch.randn_like(ref.weight), torch.randn_like(ref.bias)
        lin.weight.main_grad.copy_(gw)
        lin.bias.main_grad.copy_(gb)
        ref.weight.grad, ref.bias.grad = gw.clone(), gb.clone()
        eng.step()
        opt.step()
    assert torch.allclose(lin.weight, ref.weight, atol=1e-6)
    assert torch.allclose(lin.bias, ref.bias, atol=1e-6)


def test_reference_adamw_formula():
    """p -= lr*sqrt(bc2)/bc1 * m/(sqrt(v/bc2)+eps); p -= lr*wd*p  (the reference's AdamW::step)."""
    p0 = torch.tensor([1.0, -2.0, 0.5])
    g = torch.tensor([0.1, -0.3, 0.2])
    mod = torch.nn.Module()
    mod.w = torch.nn.Parameter(p0.clone().view(1, 3))
    eng = FlatParamEngine(mod, lr=0.1, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, max_grad_norm=0.0, reference_formula=True)
    mod.w.main_grad.copy_(g.view(1, 3))
    eng.step()
    m, v = 0.1 * g, 0.001 * g * g
    bc1, bc2 = 0.1, 0.001
    exp = p0 - 0.1 * (bc2 ** 0.5) / bc1 * m / ((v / bc2).sqrt() + 1e-8)
    exp = exp - 0.1 * 0.01 * exp
    assert torch.allclose(mod.w.view(-1), exp, atol=1e-6)


def test_token_loader_next_token_labels():
    toks = torch.arange(0, 101)
    dl = TokenLoader(toks, batch_size=2, seq_len=10)
    assert len(dl) == 5
    ids, labels = next(iter(dl))
    assert torch.equal(labels, ids + 1)
