"""B200-native replacement for tnsr's cached GPT inference backend."""
from .nn import (Backend, Gpt, GptAttentionPrecision, GptConfig, GptDecoder, GptDecoderOptions,
                 GptPrefillMode, Parameter, TnsrError, model_parameters)

__all__ = ["Backend", "Gpt", "GptAttentionPrecision", "GptConfig", "GptDecoder", "GptDecoderOptions",
           "GptPrefillMode", "Parameter", "TnsrError", "model_parameters"]
