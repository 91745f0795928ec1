from .checkpoint import (CheckpointError, load_checkpoint, load_params_multi, save_checkpoint,  # noqa: F401
                         save_params_multi)
from .safetensors import (SafeTensors, SafeTensorsError, SafeTensorsWriter, load_safetensors,  # noqa: F401
                          save_safetensors)
from .hdf5 import H5Error, H5File, read_hdf5, write_hdf5  # noqa: F401
