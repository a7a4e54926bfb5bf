from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import pifutar  # noqa: F401  (registers Pifutar)
