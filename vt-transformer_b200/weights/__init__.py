from .loader import (DictSource, RandomSource, SafetensorsSource, WeightError, WeightSource, check_against,
                     random_tensor, register_initialiser, unregister_initialiser)
from .random_init import write_random_model
from .safetensors_io import SafetensorsError
