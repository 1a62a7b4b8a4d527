"""The benchmark workloads at smoke scale (small models of the same families) on one GPU."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [2, 3, 4])
def test_engine_workloads_smoke(n):
    from unillm_b200.benchmark import workloads as W
    from unillm_b200.ops import cuda_ops

    r = W.gpu_config(n, 0.02, (0, 1, None, "cuda:0"))
    cuda_ops.check_device_errors()
    assert r["output_tokens"] > 0 and r["tok_s_device"] > 0 and r["ttft_p50_ms"] > 0 and r["tpot_p50_ms"] > 0
    if n == 4:
        assert r["prefix_hit_tokens"] > 0


def test_decode_sweep_smoke():
    from unillm_b200.benchmark import workloads as W

    rs = W.config5(0.02, (0, 1, None, "cuda:0"))
    assert [r["batch"] for r in rs] == [1, 8] and all(r["tpot_ms"] > 0 for r in rs)
