"""Typed configurations read from a model folder's config.json."""
from .base import ConfigError, ConfigReader, architecture_name, read_config_json
from .llama4 import Llama4TextConfig, RopeScaling
from .notedra import NotedraConfig, NotedraLayer, NotedraMLP
from .gisilix import GisilixConfig, GisilixLayer, GisilixMLP, GisilixYarn
from .latinex import LatinexConfig, LatinexLayer, LatinexMoE
from .zaposun import ZaposunAttention, ZaposunConfig, ZaposunLayer, ZaposunScan

__all__ = ["ConfigError", "ConfigReader", "architecture_name", "read_config_json",
           "Llama4TextConfig", "RopeScaling", "NotedraConfig", "NotedraLayer", "NotedraMLP", "ZaposunAttention",
           "ZaposunConfig", "ZaposunLayer", "ZaposunScan", "LatinexConfig", "LatinexLayer", "LatinexMoE", "GisilixConfig", "GisilixLayer", "GisilixMLP", "GisilixYarn"]
