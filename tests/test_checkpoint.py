

def test_dense_trainer_v2_checkpoint_layout_and_roundtrip(tmp_path):
    import struct
    import torch
    from innova_b200.formats import checkpoint as ck
    path = str(tmp_path / "c.ckpt")
    params = [torch.arange(6, dtype=torch.float32).view(2, 3), torch.tensor([1.5, -2.0])]
    m = [torch.full((2, 3), 0.25), torch.zeros(2)]
    ck.save_checkpoint_v2(path, params, step=7, lr=3e-4, exp_avg=m)
    raw = open(path, "rb").read()
    assert struct.unpack_from("<IIIfI", raw, 0)[:3] == (0x4B504843, 2, 7) and abs(struct.unpack_from("<f", raw, 12)[0] - 3e-4) < 1e-9
    # first tensor record: name length 7, "param_0", payload = rank 2, dims 2 x 3, dtype 4 (fp32), 24 data bytes
    assert struct.unpack_from("<I", raw, 20)[0] == 7 and raw[24:31] == b"param_0"
    assert struct.unpack_from("<I", raw, 31)[0] == 4 + 16 + 1 + 24 and struct.unpack_from("<iqqB", raw, 35) == (2, 2, 3, 4)
    back = ck.load_checkpoint_v2(path)
    assert back["step"] == 7 and torch.equal(back["params"][0], params[0]) and torch.equal(back["exp_avg"][0], m[0])
    assert torch.equal(back["exp_avg_sq"][1], torch.zeros(2))
    open(path, "r+b").write(b"\\x00\\x00\\x00\\x00")
    import pytest
    with pytest.raises(IOError):
        ck.load_checkpoint_v2(path)


def test_trainer_v2_checkpoint_resumes_bit_exact(tmp_path):
    import torch
    from innova_b200.formats import checkpoint as ck
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.training.trainer import TrainConfig, Trainer
    torch.manual_seed(0)
    ids = torch.randint(0, 256, (2, 16))
    def make():
        return Trainer(DenseModel(PRESETS["tiny"](), dtype=torch.float32, device="cpu", seed=1), TrainConfig(lr=1e-3))
    a = make()
    for _ in range(3):
        a.train_step(ids, ids)
    ck.save_trainer_v2(a, str(tmp_path / "t.ckpt"))
    la = float(a.train_step(ids, ids))
    b = make()
    assert ck.load_trainer_v2(b, str(tmp_path / "t.ckpt")) == 3
    lb = float(b.train_step(ids, ids))
    assert abs(la - lb) < 1e-6
