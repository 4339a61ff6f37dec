import dataclasses
import json
from typing import Optional

import pytest

from khaosz_b200.config import AutoRegressiveLMConfig, BaseConfig, ConfigFactory, EncoderConfig, PipelineConfig, TrainConfig
from khaosz_b200.factory import BaseFactory, Registry


def test_registry_and_factory_basics():
    class F(BaseFactory[object]):
        pass

    class G(BaseFactory[object]):
        pass

    @F.register("a", category="x", priority=2)
    class A:
        def __init__(self, v, scale=1):
            self.v, self.scale = v, scale

    @F.register("b", category="y", priority=1)
    class B:
        def __init__(self, **kw):
            self.kw = kw

    assert F.list_registered() == ["a", "b"] and G.list_registered() == []
    assert F.is_registered("a") and not G.is_registered("a")
    obj = F.create("a", 3, scale=2, unknown=9)  # unknown kwarg filtered
    assert (obj.v, obj.scale) == (3, 2)
    assert F.create("b", unknown=9).kw == {"unknown": 9}  # **kwargs keeps everything
    assert F.list_by_category("x") == ["a"] and F.list_by_priority() == ["b", "a"]
    assert F.get_component_class("a") is A
    with pytest.raises(ValueError, match="Unknown component"):
        F.create("zzz")
    with pytest.raises(ValueError, match="already registered"):
        F.register("a")(A)
    r = Registry()
    r.register("k", int)
    with pytest.raises(KeyError):
        r.get("missing")


def test_factory_validation_hook():
    class Base:
        pass

    class F(BaseFactory[Base]):
        @classmethod
        def _validate_component(cls, c):
            if not issubclass(c, Base):
                raise TypeError("bad")

    with pytest.raises(TypeError):
        F.register("x")(int)


def test_base_config_roundtrip_and_coercion(tmp_path):
    @dataclasses.dataclass
    class Inner(BaseConfig):
        n: int = 1

    @dataclasses.dataclass
    class Outer(BaseConfig):
        a: int = 0
        b: Optional[float] = None
        inner: Inner = dataclasses.field(default_factory=Inner)
        fn: object = None

    o = Outer.from_dict({"a": 3.0, "b": 2, "inner": {"n": 5.0}, "junk": 1})
    assert o.a == 3 and isinstance(o.a, int) and o.b == 2.0 and isinstance(o.b, float) and o.inner.n == 5
    o.fn = lambda: 1
    d = o.to_dict()
    assert "fn" not in d and d["inner"] == {"n": 5}
    p = tmp_path / "c.json"
    o.to_json(p)
    assert Outer.from_json(p).inner.n == 5


def test_model_config_files_and_dispatch(tmp_path):
    cfg = AutoRegressiveLMConfig(vocab_size=10, dim=8, n_layers=1, n_heads=2, n_kv_heads=1)
    path = tmp_path / "config.json"
    cfg.to_file(str(path))
    raw = json.loads(path.read_text())
    assert "kv_lora_rank" not in raw and raw["attn_type"] == "gqa"  # None fields dropped
    assert AutoRegressiveLMConfig.from_file(str(path)).dim == 8
    assert isinstance(ConfigFactory.load(raw), AutoRegressiveLMConfig)
    assert isinstance(ConfigFactory.load({"model_type": "embedding", "dim": 4}), EncoderConfig)


def test_train_config_required_fields():
    with pytest.raises(ValueError, match="model_fn"):
        TrainConfig()
    cfg = TrainConfig(model_fn=lambda: None, strategy="seq", dataset=[1], optimizer_fn=lambda m: None,
                      scheduler_fn=lambda o: None)
    assert cfg.grad_accum_steps == 1 and cfg.metrics == ["loss", "lr"] and cfg.parallel_mode == "none"


def test_pipeline_config_defaults():
    cfg = PipelineConfig.from_dict({"input": {"sections": [{"field": "text", "action": "train"}]},
                                    "output": {"dtype": {"loss_mask": "bool"}}})
    assert cfg.preprocessing.max_seq_len == 2048 and cfg.output.storage_format == "bin"
    assert cfg.output.dtype_of("loss_mask") == "bool" and cfg.output.dtype_of("sequence") == "int32"
    assert cfg.action_for_role("user") == "mask"
