"""Architectures known to the registry.  Importing this package registers them."""

from ..config.lemesun import LemesunConfig
from ..config.losivik import LosivikConfig
from ..config.nulalorn import NulalornConfig
from ..config.qwen3 import Qwen3Config
from ..config.zigivik import ZigivikConfig
from ..registry import register_architecture

register_architecture("Qwen3ForCausalLM", Qwen3Config, model_type="qwen3")
register_architecture("Lemesun", LemesunConfig)
register_architecture("Losivik", LosivikConfig)
register_architecture("Nulalorn", NulalornConfig)
register_architecture("Zigivik", ZigivikConfig)
