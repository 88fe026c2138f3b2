from . import llama, medolorn, rekasun, rorovik, zuzadra  # noqa: F401  (register the architectures)
from .decoder import Block, DecoderModel, register_arrangement
from .llama import build_llama_spec
from .medolorn import build_medolorn_spec
from .rekasun import build_rekasun_spec
from .rorovik import build_rorovik_spec
from .zuzadra import build_zuzadra_spec

__all__ = ["Block", "DecoderModel", "build_llama_spec", "build_medolorn_spec", "build_rekasun_spec",
           "build_rorovik_spec", "build_zuzadra_spec", "register_arrangement"]
