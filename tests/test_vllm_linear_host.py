"""Host-side checks of the serving-engine Linear path (no GPU): the decode-selector parser, and -- where the reference
tree is at hand -- that every (pid, split_k) its patch names is a kernel this library has, under its K alignment."""
import os

import pytest

from moonpoly_b200 import vllm_linear

PATCH = os.path.join(os.environ.get("REFERENCE_DIR", "/root/reference"), "integrations", "vllm", "v0.10.0",
                     "moonpoly_linear.patch")


def test_decode_selector_parser(tmp_path):
    f = tmp_path / "p.patch"
    f.write_text("+_SEL = {\n+    (1, 27648, 5120): (304, 4),\n+    (16, 5120, 5120): (96, 2),\n+}\n     (9, 9, 9): (1, 1),\n")
    rows = vllm_linear.decode_selector_from_patch(str(f))
    assert rows == {(1, 27648, 5120): (304, 4), (16, 5120, 5120): (96, 2)}
    vllm_linear.load_decode_selector(rows)
    assert vllm_linear.DECODE_SELECTOR[(16, 5120, 5120)] == (96, 2)
    vllm_linear.load_decode_selector({})


@pytest.mark.skipif(not os.path.exists(PATCH), reason="reference tree not present")
def test_every_row_of_the_reference_table_names_a_kernel_here(api):
    rows = vllm_linear.decode_selector_from_patch(PATCH)
    assert len(rows) >= 20
    for (m, n, k), (pid, split_k) in rows.items():
        tile, align = api.pid_info(api.MP_FP16, pid)
        assert k % align == 0 and split_k >= 1 and tile[0] == 16, (m, n, k, pid)
        assert api.workspace_size(api.MP_FP16, pid, n, m, k, split_k) >= 0


def test_gates_need_no_gpu(monkeypatch):
    for name in ("VLLM_MOONPOLY_STREAMK_MAX_M", "VLLM_MOONPOLY_STREAMK_ALLOW_M", "VLLM_MOONPOLY_STREAMK_ALLOW_N",
                 "VLLM_MOONPOLY_STREAMK_ALLOW_K", "VLLM_USE_MOONPOLY_LINEAR"):
        monkeypatch.delenv(name, raising=False)
    assert vllm_linear.streamk_shape_allowed(1, 5120, 5120) and vllm_linear.streamk_shape_allowed(15, 27648, 13824)
    assert not vllm_linear.streamk_shape_allowed(16, 5120, 5120) and not vllm_linear.streamk_shape_allowed(1, 5119, 5120)
    monkeypatch.setenv("VLLM_MOONPOLY_STREAMK_ALLOW_K", "13824")
    assert not vllm_linear.streamk_shape_allowed(1, 5120, 5120) and vllm_linear.streamk_shape_allowed(1, 5120, 13824)
    import torch
    assert vllm_linear.apply_moonpoly_linear(torch.zeros(4, 8), torch.zeros(2, 8)) is None       # switch off: declines
