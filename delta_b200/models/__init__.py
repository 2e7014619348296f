"""Model specifications and the generic model that runs them."""
from ..config.model_config import YiConfig
from ..config.registry import register_architecture
from .model import Model
from .spec import LayerSpec, ModelSpec, RunEntry
from .yi import yi_spec
from .roletar import roletar_spec
from ..config.roletar_config import RoletarConfig
from ..parts import latent_attention, row_attention, selective_scan, streams  # noqa: F401  (register their parts)

for _name in ("LlamaForCausalLM", "YiForCausalLM"):
    register_architecture(_name, YiConfig.from_dict, yi_spec)
register_architecture("Roletar", RoletarConfig.from_dict, roletar_spec)
