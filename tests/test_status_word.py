"""The device status word is read by library code at its existing synchronisation points, not only by benchmarks."""
import pytest
import torch


def _tiny_trainer(tmp_path=None):
    from innova_b200.models import DenseModel, tiny_dense
    from innova_b200.training.trainer import Trainer, TrainConfig
    cfg = tiny_dense(num_layers=1, hidden_size=32, num_heads=1, head_dim=32, ffn_hidden_size=64, max_seq_len=8, ste_format="")
    model = DenseModel(cfg, dtype=torch.float32)
    return Trainer(model, TrainConfig(log_interval=1, max_steps=2, save_path=str(tmp_path / "m.oil") if tmp_path else "", save_interval=0))


def test_check_status_raises_clears_and_runs_reset_hooks():
    from innova_b200.ops import runtime as rt
    seen = []
    rt.on_status_error(seen.append)
    try:
        rt.status_tensor("cpu").fill_(5)
        with pytest.raises(RuntimeError, match="wait_peer"):
            rt.check_status("cpu")
        assert seen == [5]
        rt.check_status("cpu")          # cleared
    finally:
        rt._on_error.remove(seen.append) if seen.append in rt._on_error else rt._on_error.clear()


def test_trainer_reads_the_status_word_when_it_logs_and_before_it_saves(tmp_path):
    from innova_b200.ops import runtime as rt
    tr = _tiny_trainer(tmp_path)
    ids = torch.randint(0, 256, (2, 8))
    loader = [(ids, torch.roll(ids, -1, 1))] * 3
    tr.fit(loader)                       # clean word: trains
    rt.status_tensor("cpu").fill_(1)
    with pytest.raises(RuntimeError, match="wait_full"):
        tr.fit(loader)
    rt.status_tensor("cpu").fill_(5)
    with pytest.raises(RuntimeError, match="wait_peer"):
        tr.save_checkpoint(str(tmp_path / "m.oil"))
    assert not (tmp_path / "m.oil").exists()
    tr.save_checkpoint(str(tmp_path / "m.oil"))
    assert (tmp_path / "m.oil").exists()


def test_colsum_slot_is_single_use_and_matches_only_the_same_tensor():
    """The norm backward's column sums reach only the very next linear backward, and only for the very same gradient tensor."""
    import torch
    from innova_b200.ops import runtime as rt
    dx = torch.randn(6, 4)
    cs = dx.sum(0)
    rt.offer_colsum(dx, cs)
    assert rt.take_colsum(dx.view(6, 4)) is cs          # same storage, shape and version
    assert rt.take_colsum(dx) is None                   # the slot is cleared by the first taker
    rt.offer_colsum(dx, cs)
    assert rt.take_colsum(torch.randn(6, 4)) is None and rt.take_colsum(dx) is None     # a different tensor clears it too
    rt.offer_colsum(dx, cs)
    dx.mul_(2.0)                                        # modified in place since the offer: the sums are stale
    assert rt.take_colsum(dx) is None
    rt.offer_colsum(dx, cs)
    assert rt.take_colsum(dx.view(4, 6)) is None        # same memory, other shape
