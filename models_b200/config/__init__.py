from .kabanex import KabanexConfig
from .llama import ConfigError, LlamaConfig, RopeScalingConfig
from .lovurax import LovuraxConfig
from .rolevik import RolevikConfig
from .registry import (
    config_from_dict,
    known_architectures,
    load_config,
    register_architecture,
    unregister_architecture,
)
from .specs import (
    AttentionSpec,
    BlockSpec,
    DenseFeedForwardSpec,
    EmbeddingSpec,
    GatedFeedForwardSpec,
    GatedResidualBlockSpec,
    HeadSpec,
    LatentAttentionSpec,
    LayerNormSpec,
    MinGruSpec,
    ModelSpec,
    NormSpec,
    ParallelBlockSpec,
    RetentionSpec,
    RopeScalingSpec,
    RopeSpec,
    ScheduleEntry,
    SideBySideSpec,
    SigmoidAttentionSpec,
    TalkingAttentionSpec,
)
