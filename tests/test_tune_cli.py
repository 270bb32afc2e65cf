"""The tile-table check (ffn_kernel_b200.tune) without a GPU: variant selection and table layout,
with the per-variant sweep replaced by a stand-in."""
import sys

from ffn_kernel_b200 import tune


def test_table_lists_relevant_variants_and_marks_the_fastest(monkeypatch, capsys):
    calls = []

    def fake(sweep_args, env):
        calls.append((tuple(sweep_args), dict(env)))
        slow = 2.0 if env.get("FFNK_PAIR") == "1" else 1.0
        return {"ffn_gateup(routed input)": 1.5 * slow, "ffn_down": 0.9 / slow}

    monkeypatch.setattr(tune, "run_variant", fake)
    monkeypatch.setattr(sys, "argv", ["tune", "ffn", "--M", "4096", "--d", "1024", "--h", "2816"])
    tune.main()
    out = capsys.readouterr().out.strip().splitlines()
    assert out[0].startswith("| variant | ffn_gateup(routed input) | ffn_down |")
    assert calls[0][1] == {} and calls[0][0][:3] == ("ffn", "--M", "4096")
    envs = [c[1] for c in calls]
    assert {"FFNK_PERMUTE": "0"} in envs and {"FFNK_EPI_WARPS": "8"} in envs
    assert all("FFNK_LINEAR_COPY" not in e and "FFNK_WGRAD_PAIR" not in e for e in envs)   # not for a forward FFN
    pair_row = next(ln for ln in out if "FFNK_PAIR=1" in ln)
    assert "3.0000" in pair_row and "**0.4500**" in pair_row       # slower gate/up, fastest down


def test_linear_backward_adds_the_weight_gradient_variant(monkeypatch, capsys):
    envs = []
    monkeypatch.setattr(tune, "run_variant", lambda args, env: (envs.append(dict(env)), {"linear_fwd": 1.0})[1])
    monkeypatch.setattr(sys, "argv", ["tune", "linear", "--M", "4096", "--K", "1024", "--N", "1024", "--bwd"])
    tune.main()
    capsys.readouterr()
    assert {"FFNK_WGRAD_PAIR": "0"} in envs and {"FFNK_LINEAR_COPY": "0"} in envs
    assert all("FFNK_PERMUTE" not in e for e in envs)
