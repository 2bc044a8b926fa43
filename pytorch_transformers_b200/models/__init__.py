"""Architectures: each module turns its configuration into a ModelSpec and registers itself."""
from ..config.falcon import FalconConfig
from ..config.registry import register_architecture
from ..config.pafevik import PafevikConfig
from .falcon import FALCON_NAME_RULES, falcon_spec
from .pafevik import pafevik_spec
from ..config.zalunex import ZalunexConfig
from .zalunex import zalunex_spec
from ..config.pogezen import PogezenConfig
from .pogezen import pogezen_spec
from ..config.figudra import FigudraConfig
from .figudra import figudra_spec

register_architecture(
    "falcon", ("FalconForCausalLM", "RWForCausalLM"), FalconConfig, falcon_spec, name_rules=FALCON_NAME_RULES,
    aliases=("RefinedWeb", "RefinedWebModel"))  # custom-code checkpoints (convert_custom_code_checkpoint.py:35-55)

register_architecture("pafevik", ("Pafevik",), PafevikConfig, pafevik_spec)
register_architecture("zalunex", ("Zalunex",), ZalunexConfig, zalunex_spec)
register_architecture("pogezen", ("Pogezen",), PogezenConfig, pogezen_spec)
register_architecture("figudra", ("Figudra",), FigudraConfig, figudra_spec)
