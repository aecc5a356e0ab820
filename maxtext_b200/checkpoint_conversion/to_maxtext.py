"""`python -m maxtext_b200.checkpoint_conversion.to_maxtext <yml> model_name=... hf_model_path=DIR base_output_directory=OUT`

Role of src/maxtext/checkpoint_conversion/to_maxtext.py: HF safetensors -> a params-only checkpoint that `load_parameters_path` accepts.
"""
import sys

from ..config import pyconfig
from . import hf


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  src = [a.split("=", 1)[1] for a in argv if a.startswith("hf_model_path=")]
  argv = [a for a in argv if not a.startswith("hf_model_path=")]
  if not src:
    raise SystemExit("hf_model_path=<directory with *.safetensors> is required")
  config = pyconfig.initialize(argv + ["hardware=cpu"], num_devices=1)
  out = hf.convert_hf_to_checkpoint(src[0], config, config.checkpoint_dir)
  print(f"wrote {out}")


if __name__ == "__main__":
  main()
