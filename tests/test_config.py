"""Config system: dataclass decoding, choice registries, unions, codecs, YAML includes, command-line overrides."""
import dataclasses
import datetime
import enum
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import pytest
import torch

from levanter_b200 import config as C


@dataclass(frozen=True)
class Animal(C.ChoiceRegistry):
    @classmethod
    def default_choice_name(cls):
        return "dog"


@Animal.register_subclass("dog")
@dataclass(frozen=True)
class Dog(Animal):
    legs: int = 4
    name: str = "rex"


@Animal.register_subclass("bird")
@dataclass(frozen=True)
class Bird(Animal):
    wingspan: float = 0.3


class Color(str, enum.Enum):
    red = "red"
    blue = "blue"


@dataclass
class Inner:
    x: int = 1
    ratio: float = 0.5
    tags: List[str] = field(default_factory=list)


@dataclass
class Outer:
    inner: Inner = field(default_factory=Inner)
    pet: Animal = field(default_factory=Dog)
    maybe: Optional[int] = None
    either: Union[int, str] = 0
    color: Color = Color.red
    where: Path = Path("logs")
    every: datetime.timedelta = datetime.timedelta(minutes=15)
    table: Dict[str, float] = field(default_factory=dict)
    pair: Tuple[int, int] = (0, 0)
    mp: C.Policy = field(default_factory=lambda: C.Policy.parse("f32"))


def test_defaults_and_nested_decode():
    o = C.decode(Outer, {})
    assert o.inner.x == 1 and isinstance(o.pet, Dog) and o.where == Path("logs")
    o = C.decode(Outer, {"inner": {"x": 3, "tags": ["a", "b"]}, "maybe": 5, "either": "s", "color": "blue", "where": "/tmp/x",
                         "every": "1h30m", "table": {"a": 1}, "pair": [2, 3]})
    assert o.inner == Inner(3, 0.5, ["a", "b"]) and o.maybe == 5 and o.either == "s" and o.color is Color.blue
    assert o.where == Path("/tmp/x") and o.every == datetime.timedelta(minutes=90) and o.table == {"a": 1.0} and o.pair == (2, 3)


def test_choice_registry_type_key_and_default():
    assert isinstance(C.decode(Outer, {"pet": {"type": "bird", "wingspan": 1.5}}).pet, Bird)
    assert C.decode(Outer, {"pet": {"legs": 3}}).pet == Dog(legs=3)  # no type key: the default choice
    with pytest.raises(C.ConfigError):
        C.decode(Outer, {"pet": {"type": "fish"}})
    assert Animal.get_choice_class("bird") is Bird


def test_unknown_key_and_bad_type_are_errors_with_path():
    with pytest.raises(C.ConfigError) as e:
        C.decode(Outer, {"inner": {"y": 1}})
    assert "inner" in str(e.value) and "y" in str(e.value)
    with pytest.raises(C.ConfigError):
        C.decode(Outer, {"inner": {"x": "not a number"}})


def test_policy_parsing():
    p = C.Policy.parse("p=f32,c=bfloat16")
    assert p.param_dtype == torch.float32 and p.compute_dtype == torch.bfloat16
    assert C.decode(Outer, {"mp": "bf16"}).mp.compute_dtype == torch.bfloat16


def test_encode_round_trip_and_yaml():
    o = C.decode(Outer, {"pet": {"type": "bird"}, "color": "blue", "every": "2h", "where": "/x"})
    enc = C.encode(o)
    assert enc["pet"]["type"] == "bird" and enc["color"] == "blue" and enc["where"] == "/x"
    again = C.decode(Outer, enc)
    assert again.pet == o.pet and again.every == o.every and again.color == o.color
    assert "wingspan" in C.to_yaml(o)


def test_yaml_include_and_overrides(tmp_path):
    (tmp_path / "base.yaml").write_text("x: 7\nratio: 0.25\n")
    (tmp_path / "main.yaml").write_text("inner: !include base.yaml\nmaybe: 2\n")
    o = C.parse(Outer, str(tmp_path / "main.yaml"), args=["--inner.x", "9", "--pet.type", "bird", "--pet.wingspan=2.5", "--color", "blue"])
    assert o.inner.x == 9 and o.inner.ratio == 0.25 and o.maybe == 2 and o.pet == Bird(2.5) and o.color is Color.blue


def test_multiple_config_files_merge(tmp_path):
    (tmp_path / "a.yaml").write_text("inner: {x: 2}\nmaybe: 1\n")
    (tmp_path / "b.yaml").write_text("inner: {ratio: 0.9}\n")
    o = C.parse(Outer, [str(tmp_path / "a.yaml"), str(tmp_path / "b.yaml")], args=[])
    assert o.inner.x == 2 and o.inner.ratio == 0.9 and o.maybe == 1


def test_main_decorator_finds_config_path(tmp_path):
    (tmp_path / "c.yaml").write_text("maybe: 4\n")
    seen = {}

    def fn(cfg: Outer):
        seen["cfg"] = cfg

    C.main(fn, args=["--config_path", str(tmp_path / "c.yaml"), "--inner.x", "11"])()
    assert seen["cfg"].maybe == 4 and seen["cfg"].inner.x == 11


def test_negative_numbers_and_lists_on_command_line():
    over = C.parse_overrides(["--a.b", "-3", "--c", "[1, 2]", "--flag", "true", "--name", "x y"])
    assert over == {"a": {"b": -3}, "c": [1, 2], "flag": True, "name": "x y"}


# ---------------------------------------------------------------- scenarios after the reference's tests/test_config.py
def test_main_decorator_reads_a_config_from_an_fsspec_url_with_overrides():
    import dataclasses as dc

    import fsspec

    from levanter_b200 import config as C

    with fsspec.open("memory://lvb_cfg/test.yaml", "w") as f:
        f.write("project: test\n")

    @dc.dataclass
    class Config:
        project: str
        x: int = 1

    seen = {}

    @C.main(args=["--config_path", "memory://lvb_cfg/test.yaml", "--x", "2"])
    def main(config: Config):
        seen["cfg"] = config

    main()
    assert seen["cfg"].project == "test" and seen["cfg"].x == 2


def test_trainer_axis_mappings_follow_tensor_parallel_axes():
    from levanter_b200.trainer import TrainerConfig

    cfg = TrainerConfig(tensor_parallel_axes=["a1", "a2"])
    assert cfg.tensor_parallel_axes == ["a1", "a2"]
    assert cfg.compute_axis_mapping == {"batch": ("replica", "data"), "a1": "model", "a2": "model"}
    assert cfg.parameter_axis_mapping == {"embed": "data", "a1": "model", "a2": "model", "batch": ("replica", "data")}


def test_dataset_configs_decode_from_yaml_through_the_main_decorator():
    import dataclasses as dc

    import fsspec

    from levanter_b200 import config as C
    from levanter_b200.data.text import HfDatasetSourceConfig, HfSingleDatasetLMConfig, LMMixtureDatasetConfig, UrlDatasetSourceConfig

    @dc.dataclass
    class Single:
        data: HfSingleDatasetLMConfig = dc.field(default_factory=HfSingleDatasetLMConfig)

    @dc.dataclass
    class Mixture:
        data: LMMixtureDatasetConfig = dc.field(default_factory=LMMixtureDatasetConfig)

    with fsspec.open("memory://lvb_cfg/single.yaml", "w") as f:
        f.write('data:\n  id: dlwh/wikitext_103_detokenized\n  cache_dir: "gs://levanter-data/tokenized/wikitext"\n')
    with fsspec.open("memory://lvb_cfg/mixture.yaml", "w") as f:
        f.write("""
data:
  configs:
    owt:
      train_urls:
        - "gs://pubmed-mosaic/openwebtext-sharded/openwebtext_train.{1..128}-of-128.jsonl.gz"
      validation_urls:
        - "gs://pubmed-mosaic/openwebtext-sharded/openwebtext_val.{1..8}-of-8.jsonl.gz"
    wikitext:
      id: dlwh/wikitext_103_detokenized
  train_weights:
    owt: 0.6
    wikitext: 0.4
  tokenizer: gpt2
  cache_dir: "gs://levanter-data/tokenized/mixture"
""")
    seen = {}

    @C.main(args=["--config_path", "memory://lvb_cfg/single.yaml"])
    def one(config: Single):
        seen["single"] = config

    @C.main(args=["--config_path", "memory://lvb_cfg/mixture.yaml"])
    def two(config: Mixture):
        seen["mixture"] = config

    one()
    two()
    assert seen["single"].data.id == "dlwh/wikitext_103_detokenized" and seen["single"].data.cache_dir == "gs://levanter-data/tokenized/wikitext"
    mix = seen["mixture"].data
    assert mix.train_weights == {"owt": 0.6, "wikitext": 0.4} and mix.tokenizer == "gpt2"
    assert isinstance(mix.configs["owt"], UrlDatasetSourceConfig) and isinstance(mix.configs["wikitext"], HfDatasetSourceConfig)
    assert len(mix.configs["owt"].urls_for_split("validation")) == 1 and mix.configs["wikitext"].id == "dlwh/wikitext_103_detokenized"


def test_custom_codecs_and_precision_policy_casts():
    import dataclasses as dc
    import fractions

    import torch

    from levanter_b200 import config as C

    C.register_codec(fractions.Fraction, lambda v: fractions.Fraction(str(v)), lambda f: f"{f.numerator}/{f.denominator}")

    @dc.dataclass
    class Holder:
        ratio: fractions.Fraction = fractions.Fraction(1, 2)
        mp: C.Policy = dc.field(default_factory=lambda: C.Policy.parse("f32"))

    h = C.decode(Holder, {"ratio": "3/4", "mp": "p=f32,c=bfloat16,o=f32"})
    assert h.ratio == fractions.Fraction(3, 4) and C.encode(h)["ratio"] == "3/4"
    assert C.encode(h)["mp"] == "compute=bfloat16,params=float32,output=float32"
    assert C.decode(Holder, C.encode(h)) == h  # what is written can be read back

    p = h.mp
    x = torch.ones(2, dtype=torch.float32)
    ids = torch.ones(2, dtype=torch.int32)
    assert p.cast_to_compute(x).dtype == torch.bfloat16 and p.cast_to_param(x.bfloat16()).dtype == torch.float32 and p.cast_to_output(x.bfloat16()).dtype == torch.float32
    assert p.cast_to_compute(ids).dtype == torch.int32  # integers are left alone
    assert C.Policy.parse("bfloat16") == C.Policy(torch.bfloat16, torch.bfloat16, torch.bfloat16)
    assert C.Policy.parse("compute=bfloat16,params=float32").output_dtype == torch.bfloat16  # the output follows the compute dtype
    with pytest.raises(C.ConfigError):
        C.Policy.parse("q=f32")
