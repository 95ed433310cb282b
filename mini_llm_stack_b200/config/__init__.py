from .model_config import (ConfigError, DenseLlamaConfig, canonical_dtype_name,
                           read_config_json, write_config_json)
from .engine_options import EngineOptions
from .registry import (register_architecture, unregister_architecture,
                       lookup_architecture, architecture_names, config_from_dict,
                       config_from_folder, build_model)
