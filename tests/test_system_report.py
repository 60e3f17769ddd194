"""Machine / network report: runs on any box, reads only; GPU section against a stand-in for NVML."""
import socket

from adaptivetrainingsystem_b200.utils import system_report as R


class _FakeNvml:
    NVML_CLOCK_SM, NVML_TEMPERATURE_GPU, NVML_NVLINK_MAX_LINKS = 1, 0, 18
    calls = []

    class _Mem:
        total, used = 183359 * 2 ** 20, 5 * 2 ** 30

    def nvmlInit(self): self.calls.append("init")
    def nvmlShutdown(self): self.calls.append("shutdown")
    def nvmlDeviceGetCount(self): return 8
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetName(self, h): return b"NVIDIA B200"
    def nvmlDeviceGetMemoryInfo(self, h): return self._Mem
    def nvmlDeviceGetCudaComputeCapability(self, h): return (10, 0)
    def nvmlDeviceGetClockInfo(self, h, k): return 1500
    def nvmlDeviceGetMaxClockInfo(self, h, k): return 1965
    def nvmlDeviceGetEnforcedPowerLimit(self, h): return 1000000
    def nvmlDeviceGetTemperature(self, h, k): return 41
    def nvmlDeviceGetNvLinkState(self, h, l): return 1

    def __getattr__(self, name):            # anything that would CHANGE a setting is a test failure
        raise AssertionError(f"unexpected NVML call {name}")


def test_machine_report_and_recommendation():
    fake = _FakeNvml()
    rep = R.native_properties(nvml=fake)
    assert rep["cpu"]["logical_cores"] and rep["memory"]["total_gb"] > 0 and rep["software"]["python"]
    assert len(rep["gpus"]) == 8 and rep["gpus"][0]["nvlink_active_links"] == 18 and rep["gpus"][0]["capability"] == "10.0"
    assert fake.calls == ["init", "shutdown"]
    rec = rep["recommended"]
    assert rec["preset"] == "mixtral_8x7b" and rec["precision"] == "mixed_bf16" and rec["expert_parallel_size"] == 8 and rec["native_kernels"]
    assert R.recommend([], {})["preset"] == "debug"
    assert R.recommend([{"memory_gb": 40.0, "capability": "8.0"}], {})["native_kernels"] is False


def test_network_report_finds_ports_and_opens_a_store():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        s.listen(1)
        taken = s.getsockname()[1]
        assert not R.port_free(taken)
        assert R.reachable("127.0.0.1", taken) is not None
        rep = R.network_report(master_port=taken)
        assert rep["ports_free"][taken] is False and any("is taken" in a for a in rep["advice"])
    assert rep["rendezvous"]["ok"] and rep["ready_single_node"]
    assert any(i["name"] == "lo" for i in rep["interfaces"])
    assert R.main(["--network", "--json"]) == 0


def test_rank_recorder_merges_ranks_and_tensor_detector_sees_allocations(tmp_path):
    import time
    import torch
    from adaptivetrainingsystem_b200.utils.debug_tools import RankRecorder, TensorDetector, timeline_text
    d = str(tmp_path / "rec")
    for rank in (0, 1):
        r = RankRecorder(rank, d)
        with r.record("forward"):
            time.sleep(0.002)
        with r.record("backward"):
            time.sleep(0.001)
        assert r.export().endswith(f"rank_{rank}.json")
    events = RankRecorder.merge(d)
    assert len(events) == 4 and events[0]["start"] == 0.0 and {e["rank"] for e in events} == {0, 1}
    assert all(e["end"] >= e["start"] for e in events)
    text = timeline_text(events, 40)
    assert text.count("rank") == 2 and "A=backward" in text and "B=forward" in text
    det = TensorDetector(include_cpu=True)
    det.detect()
    keep = torch.zeros(1000, 3)
    rep = det.detect()
    assert any(shape == (1000, 3) for _, shape, _, _ in rep["new"]) and rep["bytes_per_device"]["cpu"] >= 12000
    del keep
    assert any(shape == (1000, 3) for _, shape, _, _ in det.detect()["gone"])
