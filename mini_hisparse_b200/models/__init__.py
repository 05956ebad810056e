from . import dotivik, koronex, qwen2, rizovik, tudasun  # noqa: F401  (register Dotivik, Koronex, Qwen2ForCausalLM, Rizovik and Tudasun)
from .decoder import DecoderModel
