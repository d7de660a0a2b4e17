"""Typed configuration and the architecture registry."""
from .registry import ConfigError, load_config, parse_config, register_architecture, registered_architectures
from .specs import (AttentionSpec, DenseMLPSpec, GatedLinearAttentionSpec, HyperConnectionSpec, LayerSpec,
                    Llama3RopeScaling, MatrixLSTMSpec, ModelConfig, NoPositionSpec, RMSNormSpec, RopeSpec, RoutedFFNSpec, ScheduleEntry,
                    SinusoidalEmbeddingSpec, SwiGLUSpec, YarnRopeScaling)
from ..models import dense_decoder as _dense_decoder  # noqa: F401  (registers Llama and Qwen2)
from ..models import gafulix as _gafulix  # noqa: F401  (registers Gafulix)
from ..models import fuvevik as _fuvevik  # noqa: F401  (registers Fuvevik)
from ..models import zigipel as _zigipel  # noqa: F401  (registers Zigipel)
from ..models import vubotar as _vubotar  # noqa: F401  (registers Vubotar)
