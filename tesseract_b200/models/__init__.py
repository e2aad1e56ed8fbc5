"""Architectures; importing this package registers them."""

from . import kazodra, ladedra, llama, pekodra, revesun  # noqa: F401  (registration)
from .decoder import DecoderModel, expected_tensors, tensor_roles
from .llama_config import LlamaConfig, RopeScaling
from .revesun_config import RevesunConfig
from .kazodra_config import KazodraConfig
from .ladedra_config import LadedraConfig
from .pekodra_config import PekodraConfig
