from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import sozilix  # noqa: F401  (registers Sozilix)
from . import muvorax  # noqa: F401  (registers Muvorax)
from . import belasun  # noqa: F401  (registers Belasun)
