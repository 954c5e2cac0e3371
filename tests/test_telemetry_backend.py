import torch

from innova_b200.utils import backend as B
from innova_b200.utils import telemetry as T


def test_sops_and_counters():
    assert T.sops(1000, 1.0, "OIL32") == 1000 and T.sops(1000, 1.0, "OIL4") == 8000 and abs(T.info_weight("SPARK_Q0") - 21.333) < 1e-2
    c = T.SopsCounters()
    seen = []
    c.register_hook("training", lambda ph, n, s: seen.append(n))
    c.record("training", 500, 0.5)
    with c.measure("inference", 100):
        pass
    assert seen == [500] and c.rate("training", "OIL8") == 500 * 4 / 0.5 and c.rate("quantize") == 0.0
    s = T.SopsScheduler()
    s.submit(lambda: "low", 0)
    s.submit(lambda: "high", 5)
    s.submit(lambda: "low2", 0)
    assert s.run_all() == ["high", "low", "low2"]


def test_kernel_timer_and_metrics():
    kt = T.KernelTimer()
    a = torch.randn(64, 64)
    for _ in range(3):
        with kt.region("matmul", flops=2 * 64 ** 3):
            a @ a
    p = kt.summary()["matmul"]
    assert p.calls == 3 and p.total_ms > 0 and "matmul" in kt.dump()
    assert T.max_over_ranks_ms(1.5) == 1.5
    m = T.MoEMetrics(4)
    m.update(torch.tensor([10, 0, 5, 5]))
    s = m.summary()
    assert s["dead_experts"] == 1 and s["imbalance"] == 2.0 and s["entropy"] < s["max_entropy"] and "e1 " in m.histogram()
    sm = T.ServerMetrics()
    for i in range(100):
        sm.observe(i / 100, tokens=2, error=i == 0)
    assert sm.percentile(0.5) == 0.5 and 'quantile="0.99"' in sm.prometheus() and "errors_total 1" in sm.prometheus()


def test_backend_probe_and_selection():
    info = B.probe_hardware()
    assert info.cpu_count >= 1
    assert B.select_optimal_backend(B.HardwareInfo()) == "cpu"
    gpu = B.HardwareInfo(gpu_count=8, gpu_sm=100, gpu_memory_bytes=180 << 30, native_kernels=True)
    assert B.select_optimal_backend(gpu) == "cuda_sm100" and B.select_optimal_backend(gpu, model_bytes=400 << 30) == "distributed"
    gpu.world_size = 8
    assert B.select_optimal_backend(gpu) == "distributed"
    r = B.benchmark_operation(lambda: torch.randn(32, 32) @ torch.randn(32, 32), iters=3, warmup=1)
    assert r["min_ms"] <= r["median_ms"]


def test_cycle_counter_sections():
    import time
    from innova_b200.utils.telemetry import CycleCounter
    c = CycleCounter()
    for _ in range(2):
        with c.section("nap"):
            time.sleep(0.02)
    r = c.report()["nap"]
    assert r["calls"] == 2 and 0.03 < r["seconds"] < 0.5 and c.hz > 1e6
