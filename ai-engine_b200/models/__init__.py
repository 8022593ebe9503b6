from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import pifutar  # noqa: F401  (registers Pifutar)
from . import zupitar  # noqa: F401  (registers Zupitar)
from . import tizodra  # noqa: F401  (registers Tizodra)
