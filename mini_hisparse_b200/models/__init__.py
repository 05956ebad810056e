from . import dotivik, koronex, qwen2, tudasun  # noqa: F401  (register Dotivik, Koronex, Qwen2ForCausalLM and Tudasun)
from .decoder import DecoderModel
