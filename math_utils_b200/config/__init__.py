"""Typed configurations and the architecture registry."""
from .base import (ConfigError, KeyReader, LayerSpec, ModelPlan, PartSpec,
                   ScheduleEntry, default_schedule)
from .forisun import ForisunConfig
from .gpt2 import Gpt2Config
from .lusalorn import LusalornConfig
from .seledra import SeledraConfig
from .tibopel import TibopelConfig
from .registry import (Architecture, architecture_for, known_architectures,
                       load_config, read_config_json, register_architecture)

register_architecture(Architecture(
    names=("gpt2", "GPT2LMHeadModel"),
    config_class=Gpt2Config,
    # some checkpoints keep every tensor under "transformer."
    name_prefixes=("", "transformer."),
), replace=True)

register_architecture(Architecture(names=("Forisun", "forisun"), config_class=ForisunConfig), replace=True)
register_architecture(Architecture(names=("Lusalorn", "lusalorn"), config_class=LusalornConfig), replace=True)
register_architecture(Architecture(names=("Seledra", "seledra"), config_class=SeledraConfig), replace=True)
register_architecture(Architecture(names=("Tibopel", "tibopel"), config_class=TibopelConfig), replace=True)

__all__ = [
    "Architecture", "ConfigError", "ForisunConfig", "Gpt2Config", "KeyReader", "LayerSpec", "LusalornConfig", "ModelPlan",
    "PartSpec", "ScheduleEntry", "SeledraConfig", "TibopelConfig", "architecture_for", "default_schedule",
    "known_architectures", "load_config", "read_config_json", "register_architecture",
]
