from .loader import check_against, load_tensors  # noqa: F401
from .random_init import RandomSource, write_model_folder  # noqa: F401
from .safetensors import SafetensorsFolder, write_safetensors  # noqa: F401
