"""One import for the public API (counterpart of ``rustllm_core::prelude``, src/lib.rs:113-157)."""
from .core.config import (ConfigBuilder, ConfigStore, ConfigValue, Configurable, ParallelConfig,  # noqa: F401
                          PluginConfigManager)
from .core.model import (Attention, BasicGenerationConfig, BasicModelConfig, BatchedModel,  # noqa: F401
                         DecoderConfig, DiffusionSampler, ForwardModel, GenerationConfig,
                         GenerativeModel, Layer, Loss, Model, ModelBuilder, ModelConfig, MSELoss,
                         NoiseSchedule, OptimizerState, PersistentModel, QuantizableModel, Tensor,
                         TrainableModel, Transformer250MConfig)
from .core.plugin import (ModelBuilderPlugin, ModelLoaderPlugin, Plugin, PluginBuilder,  # noqa: F401
                          PluginCapabilities, PluginEntry, PluginState, TokenizerPlugin)
from .core.serialization import (ModelHeader, ModelMetadata, ModelSerializable,  # noqa: F401
                                 ParameterSerializer, calculate_checksum)
from .core.tokenizer import (PaddingStrategy, PositionedToken, StringToken, Token, Tokenizer,  # noqa: F401
                             TokenizerConfig, TruncationStrategy, VocabularyTokenizer)
from .core.traits import (Checkpoint, Component, ComponentInfo, HealthCheck, Identity, Lifecycle,  # noqa: F401
                          Metadata, Metrics, Piped, Pipeline, Process, Serialize, Validate,
                          Versioned)
from .domain.inference import InferenceRequest, InferenceResult, InferenceService  # noqa: F401
from .domain.persistence import SerializationFormat, StorageBackend  # noqa: F401
from .domain.training import TrainingConfig, TrainingEvent, TrainingService  # noqa: F401
from .foundation.error import (CommError, CompositeError, ConfigError, DeviceError, Error,  # noqa: F401
                               ErrorContext, IoError, PluginError, ProcessingError, ResourceError,
                               error_context, internal_error, invalid_input, limit_exceeded,
                               not_initialized)
from .foundation.iterator import (Iter, IteratorExt, SliceWindows, Zipper, slice_windows,  # noqa: F401
                                  slice_windows_step)
from .foundation.memory import (Arena, BumpAllocator, CowStr, MemoryStats, Pool, Rope,  # noqa: F401
                                SliceView, StringInterner, TokenBufferPool, TrackingArena,
                                ZeroCopyStringBuilder)
from .foundation.types import DType, PluginName, Shape, Version  # noqa: F401
from .plugins import PluginEvent, PluginInfo, PluginManager, PluginRegistry, PluginRegistryBuilder  # noqa: F401
from .plugins.builtin import (BasicLoaderPlugin, BasicModelPlugin, BasicTokenizerPlugin,  # noqa: F401
                              BpeTokenizerPlugin, TransformerModel, TransformerModelPlugin,
                              WordPieceTokenizerPlugin)

VERSION = Version(0, 1, 0)
NAME = "coeus_b200"
