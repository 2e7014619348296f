"""Model specifications and the generic model that runs them."""
from ..config.model_config import YiConfig
from ..config.registry import register_architecture
from .model import Model
from .spec import LayerSpec, ModelSpec, RunEntry
from .yi import yi_spec
from .roletar import roletar_spec
from .pibalorn import pibalorn_spec
from ..config.roletar_config import RoletarConfig
from ..config.pibalorn_config import PibalornConfig
from ..parts import (decay_attention, experts, latent_attention, residual, row_attention, selective_scan,  # noqa: F401
                     streams)  # (register their parts)

for _name in ("LlamaForCausalLM", "YiForCausalLM"):
    register_architecture(_name, YiConfig.from_dict, yi_spec)
register_architecture("Roletar", RoletarConfig.from_dict, roletar_spec)
register_architecture("Pibalorn", PibalornConfig.from_dict, pibalorn_spec)
