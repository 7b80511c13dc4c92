from .loader import WeightsError, load_weights, expected_disk_tensors, iter_param_decls
from .random_init import (write_random_model, random_state_dict, build_model_from_config_dict,
                          init_random_on_device)
