from .base import Reader, read_config_json
from .lfm2 import Lfm2Config
from .registry import (Architecture, architecture, config_from_dict, load_config,
                       register_architecture, registered_architectures)
