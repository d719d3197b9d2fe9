"""Config layer: dataclass <- yaml <- CLI merge, struct errors, type coercion, shipped YAMLs."""
import glob
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import pytest

from lingua_b200 import config as C

ROOT = Path(__file__).resolve().parent.parent


@dataclass
class Inner:
    dim: int = 8
    lr: float = 3e-4
    name: Optional[str] = None


@dataclass
class Outer:
    steps: int = 10
    inner: Inner = field(default_factory=Inner)
    tags: List[str] = field(default_factory=list)
    sources: Dict[str, float] = field(default_factory=dict)
    eval: Optional[Any] = None


def test_cli_dotlist_and_types():
    cli = C.from_cli(["inner.dim=32", "inner.lr=1e-3", "tags=[a,b]", "steps=100_000", "sources.x=2"])
    cfg = C.dataclass_from_dict(Outer, cli)
    assert cfg.inner.dim == 32 and cfg.inner.lr == 1e-3 and cfg.tags == ["a", "b"]
    assert cfg.steps == 100000 and cfg.sources == {"x": 2.0}


def test_struct_mode_rejects_typos():
    with pytest.raises(C.ConfigError):
        C.dataclass_from_dict(Outer, {"inner": {"dmi": 3}})
    assert C.dataclass_from_dict(Outer, {"inner": {"dmi": 3}}, strict=False).inner.dim == 8
    with pytest.raises(C.ConfigError):
        C.dataclass_from_dict(Outer, {"steps": "many"})


def test_yaml_then_cli_precedence_and_roundtrip(tmp_path):
    y = tmp_path / "c.yaml"
    y.write_text("steps: 5\ninner:\n  dim: 16\n  lr: 3e-4\neval:\n  anything: [1, 2]\n")
    cfg = C.config_from_cli(Outer, [f"config={y}", "inner.dim=64"])
    assert cfg.steps == 5 and cfg.inner.dim == 64 and cfg.inner.lr == 3e-4 and cfg.eval == {"anything": [1, 2]}
    C.dump_config(cfg, str(tmp_path / "out.yaml"), log_config=False)
    again = C.load_config_file(str(tmp_path / "out.yaml"), Outer)
    assert C.dataclass_to_dict(again) == C.dataclass_to_dict(cfg)
    assert C.flatten_dict({"a": {"b": 1, "c": {"d": 2}}}, sep="/") == {"a/b": 1, "a/c/d": 2}


@pytest.mark.parametrize("path", sorted(glob.glob(str(ROOT / "apps" / "main" / "configs" / "*.yaml"))))
def test_shipped_main_configs_load(path):
    from apps.main.train import TrainArgs

    if path.endswith("eval.yaml"):
        from apps.main.eval import EvalArgs

        C.dataclass_from_dict(EvalArgs, C.load_yaml(path))
        return
    cfg = C.dataclass_from_dict(TrainArgs, C.load_yaml(path))
    assert cfg.model.dim > 0 and cfg.data.seq_len > 0
