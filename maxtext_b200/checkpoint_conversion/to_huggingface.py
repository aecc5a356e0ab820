"""`python -m maxtext_b200.checkpoint_conversion.to_huggingface <yml> model_name=... load_parameters_path=CKPT/STEP hf_output_path=DIR`

Role of src/maxtext/checkpoint_conversion/to_huggingface.py: checkpoint -> `model.safetensors` + `config.json`.
"""
import sys

from ..config import pyconfig
from . import hf


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  dst = [a.split("=", 1)[1] for a in argv if a.startswith("hf_output_path=")]
  argv = [a for a in argv if not a.startswith("hf_output_path=")]
  if not dst:
    raise SystemExit("hf_output_path=<directory> is required")
  config = pyconfig.initialize(argv + ["hardware=cpu"], num_devices=1)
  if not config.load_parameters_path:
    raise SystemExit("load_parameters_path=<checkpoint step directory> is required")
  print(f"wrote {hf.convert_checkpoint_to_hf(config.load_parameters_path, config, dst[0])}")


if __name__ == "__main__":
  main()
