from .decl import TensorDecl
from .loader import WeightError, load_weights
from .random_init import draw, write_random_model
from .safetensors_io import SafetensorsError, index_model_dir, read_header, write_file
