from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import kikalix  # noqa: F401  (registers Kikalix)
from . import pibuvik  # noqa: F401  (registers Pibuvik)
from . import norevik  # noqa: F401  (registers Norevik)
