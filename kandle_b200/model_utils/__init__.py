"""Mirror of `@kandle/model-utils` for the models on the hot path (Qwen3, Whisper encoder)."""
from .qwen3 import (GroupedQueryAttention, Qwen3Config, Qwen3DecoderLayer, Qwen3ForCausalLM, Qwen3Model,  # noqa: F401
                    RotaryEmbedding, StaticKVCache, SwiGLUMLP, applyRotaryPosEmbDirect)
from .whisper import ResidualAttentionBlock, WhisperAudioEncoder, WhisperConfig, WhisperTextDecoder  # noqa: F401
from .sampling import SampleResult, SamplerConfig, sample, sampleGreedy  # noqa: F401
