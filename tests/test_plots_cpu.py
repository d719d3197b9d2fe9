"""apps/plots: metrics loader and the probe animation page, on files written by the library itself."""
import json

import torch

from apps.plots import analysis, probe_animation
from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs
from lingua_b200.probe import AutoProbeD


def test_metrics_frame_and_plot(tmp_path):
    run = tmp_path / "run_a"
    run.mkdir()
    (run / "config.yaml").write_text("name: run_a\noptim:\n  lr: 0.001\n")
    with open(run / "metrics.jsonl", "w") as f:
        for step in range(1, 6):
            f.write(json.dumps({"global_step": step, "loss": {"out": 5.0 / step}, "speed": {"wps": 1000.0}}) + "\n")
        f.write("{broken\n")
    df = analysis.get_merged_df(str(tmp_path / "**" / "metrics.jsonl"))
    assert len(df) == 5
    assert df["params/optim/lr"].iloc[0] == 0.001 and df["metrics/loss/out"].iloc[-1] == 1.0
    out = analysis.plot_metric(df, "loss/out", out=str(tmp_path / "loss.svg"))
    text = open(out).read()
    assert "<svg" in text or "plotly" in text


def test_probe_animation_page(tmp_path):
    torch.manual_seed(0)
    args = LMTransformerArgs(dim=32, n_layers=3, n_heads=2, vocab_size=64, max_seqlen=16)
    m = LMTransformer(args)
    m.init_weights()
    folder = tmp_path / "probe"
    folder.mkdir()
    tok = torch.randint(0, 64, (2, 17))
    for step in range(3):
        with AutoProbeD(m, str(folder / f"probe.{step}.jsonl")) as probe:
            probe.metadata = {"global_step": step}
            m(tok[:, :-1], tok[:, 1:]).backward()
    dumps = probe_animation.load_probe_folder(folder)
    assert len(dumps) == 3 and probe_animation.num_layers(dumps[0]) == 3
    ser = probe_animation.depth_series(dumps, "layers.{}.attention.wo::out")
    assert len(ser["frames"]) == 3 and all(q is not None for q in ser["frames"][0])
    out = probe_animation.render([str(folder)], ["layers.{}.attention.wo::out", "layers.{}.feed_forward.w2::w.g"],
                                 str(tmp_path / "out" / "probe.html"))
    page = open(out).read()
    assert "layers.{}.attention.wo::out" in page and "<script>" in page
