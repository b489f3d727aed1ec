from .lfm2 import ConfigError, Lfm2Config
from .registry import (architecture_name, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .specs import (AttentionSpec, LayerSpec, ModelSpec, NoPositionSpec, RMSNormSpec, RopeSpec,
                    ScheduleEntry, ShortConvSpec, SwiGLUSpec)
