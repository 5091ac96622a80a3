from .lfm2 import ConfigError, Lfm2Config
from .metanex import MetanexConfig
from .rofulorn import RofulornConfig
from .fuzelorn import FuzelornConfig
from .registry import (architecture_name, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .specs import (AttentionSpec, DistanceBiasSpec, GatedDeltaSpec, InputConvSpec, MLPSpec, SideBySideSpec, TokenPairSpec, LatentAttentionSpec, LayerNormSpec, LayerSpec, MappedAttentionSpec, ModelSpec,
                    MoESpec, NoPositionSpec,
                    RMSNormSpec, RetentionSpec, RopeSpec, ScalarRMSNormSpec, ScheduleEntry, ShortConvSpec, SwiGLUSpec,
                    TokenSideSpec)
