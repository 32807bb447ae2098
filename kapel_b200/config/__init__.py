"""Typed configurations, the model-as-data records, and the architecture registry."""
from .fusitar import FusitarConfig
from .gemma2 import ConfigError, Gemma2Config
from .kofutar import KofutarConfig
from .lokedra import LokedraConfig
from .teluzen import TeluzenConfig
from .registry import (
    architectures,
    config_class_for,
    config_from_dir,
    config_from_json,
    presets,
    read_config_file,
    register_architecture,
    unregister_architecture,
)
from .spec import (
    AttentionSpec,
    BlockSpec,
    DeltaSpec,
    EmbedSpec,
    ForgetGateSpec,
    GatedMLPSpec,
    GeneralDeltaSpec,
    HeadSpec,
    InputAddSpec,
    InputMixSpec,
    LatentAttentionSpec,
    MLPSpec,
    MLSTMSpec,
    ModelSpec,
    MoESpec,
    NormSpec,
    ParallelMixerSpec,
    PositionSpec,
    RopeScaling,
    ScheduleEntry,
    default_schedule,
)
