"""Serving: resident inference engine bindings, generation loop, HTTP endpoints."""
from .engine import (EngineConfig, EngineError, ResidentEngine, Sampling, resident_inference_abi_version,
                     resident_inference_capabilities)

__all__ = ["EngineConfig", "EngineError", "ResidentEngine", "Sampling", "resident_inference_abi_version",
           "resident_inference_capabilities"]

from .chat import (AssistantResponse, ByteTextCodec, ChatConfigurationError, ChatMessage, ChatRenderer, HuggingFaceTokenizerJSONCodec,  # noqa: E402,F401
                   IncrementalTokenDecoder, MuseGlimmerATEMRenderer, PlaceholderChatRenderer, PlainRolesRenderer, TextCodec,
                   TiktokenTextCodec, TokenIdTextCodec, load_text_codec, parse_assistant_response, resolve_chat_renderer,
                   strip_text_delimiters)
from .inference import (DFlashProposer, DraftEngineProposer, GenerationConfig, GenerationEvent, GenerationResult, InferenceError, KVCacheConfig, target_embed_and_head,  # noqa: E402,F401
                        NativeInferenceCapabilities, NativeInferenceModel, NativeInferenceSession, NativeModelLoadConfig, NGramProposer,
                        write_artifact)
