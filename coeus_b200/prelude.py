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
from .core.tokenizer import NormalizingTokenizer, SpecialTokenizer  # noqa: F401
from .core.traits import (Adapter, AsyncLifecycle, BatchProcess, Builder, Constraint, Factory,  # noqa: F401
                          FromIterator, IntoIterator, Strategy, StreamProcess)
from .domain.inference import (InferenceEvent, InferenceRequest, InferenceResult,  # noqa: F401
                               InferenceService, InferenceSession)
from .domain.modeling import (Architecture, ModelingEvent, ModelingService,  # noqa: F401
                              ModelRepository)
from .domain.modeling import ModelAggregate as DomainModelAggregate  # noqa: F401
from .domain.persistence import Checkpoint as DomainCheckpoint  # noqa: F401
from .domain.persistence import (PersistenceEvent, PersistenceService, SerializationFormat,  # noqa: F401
                                 StorageBackend)
from .domain.tokenization import Token as DomainToken  # noqa: F401
from .domain.tokenization import (TokenizationEvent, TokenizationService, TokenizerAggregate,  # noqa: F401
                                  TokenizerRepository)
from .domain.training import TrainingConfig as DomainTrainingConfig  # noqa: F401
from .domain.training import (Optimizer, TrainingConfig, TrainingEvent, TrainingService,  # noqa: F401
                              TrainingSession)
from .foundation.error import (CommError, CompositeError, ConfigError, DeviceError, Error,  # noqa: F401
                               ErrorContext, IoError, PluginError, ProcessingError, ResourceError,
                               error_context, internal_error, invalid_input, limit_exceeded,
                               not_initialized)
from .foundation.error import ContextualError, ErrorExt  # noqa: F401
from .foundation.iterator import (AdvancedIteratorExt, BatchIterator, BloomFilterBitIterator,  # noqa: F401
                                  BTreeIterator, CacheOblivious, Chunks, Iter, IteratorAdapter,
                                  IteratorExt, OwnedRopeIterator, PreciseSizeHint, Prefetch,
                                  RopeIterator, Scan, SliceWindows, StatefulIterator, StreamFusion,
                                  Stride, SuffixArrayIterator, TrieIterator, TrieNode,
                                  WaveletTreeIterator, Windows, ZeroCopySplit, ZeroCopyTokenizer,
                                  Zipper, slice_windows, slice_windows_step)
from .foundation.memory import (Arena, BumpAllocator, CowStr, LazyAlloc, MemoryStats, Pool, Rope,  # noqa: F401
                                SliceView, StringInterner, TokenBufferPool, TrackingArena,
                                ZeroCopyStringBuilder)
from .foundation.types import (BatchSize, ConfigKey, DType, DynError, HeadCount, LayerCount,  # noqa: F401
                               ModelDim, ModelDouble, ModelFloat, PluginName, SequenceLength, Shape,
                               TokenId, Version, VocabSize)
from .infer.engine import InferenceEngine  # noqa: F401
from .infer.scheduler import ContinuousBatcher  # noqa: F401
from .train.launch import ParallelRun, build_trainer  # noqa: F401
from .train.trainer import TrainConfig, Trainer  # noqa: F401
from .plugins import PluginEvent, PluginInfo, PluginManager, PluginRegistry, PluginRegistryBuilder  # noqa: F401
from .plugins.builtin import (BasicLoaderPlugin, BasicModelPlugin, BasicTokenizerPlugin,  # noqa: F401
                              BpeTokenizerPlugin, TransformerModel, TransformerModelPlugin,
                              WordPieceTokenizerPlugin)

VERSION = Version(0, 1, 0)
NAME = "coeus_b200"
