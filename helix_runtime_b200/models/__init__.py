from . import llama, rekasun  # noqa: F401  (register the architectures)
from .decoder import Block, DecoderModel, register_arrangement
from .llama import build_llama_spec
from .rekasun import build_rekasun_spec

__all__ = ["Block", "DecoderModel", "build_llama_spec", "build_rekasun_spec", "register_arrangement"]
