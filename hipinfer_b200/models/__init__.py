from .decoder import DecoderModel, StepCachePlan
from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import torirax  # noqa: F401  (registers Torirax)
from . import vegodra  # noqa: F401  (registers Vegodra)
from . import runopel  # noqa: F401  (registers Runopel)
from . import mavinex  # noqa: F401  (registers Mavinex)
from .llama import llama_spec
from .torirax import torirax_spec
from .vegodra import vegodra_spec
from .runopel import runopel_spec
from .mavinex import mavinex_spec

__all__ = ["DecoderModel", "StepCachePlan", "llama_spec", "torirax_spec", "vegodra_spec", "runopel_spec", "mavinex_spec"]
