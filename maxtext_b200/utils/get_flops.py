"""Print the training FLOPs per device per step of a configuration (src/maxtext/utils/get_flops.py):
`python -m maxtext_b200.utils.get_flops <yml> model_name=... per_device_batch_size=... max_target_length=...`."""
import json
import sys

from ..config import pyconfig
from . import flops


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  c = pyconfig.initialize(argv + ["log_config=false"] if not any(a.startswith("log_config=") for a in argv) else argv)
  total, learnable, attention = flops.training_tflops_per_device(c)
  out = {"model": c.model_name, "total_tflops_per_device_per_step": total, "learnable_weight_tflops": learnable,
         "attention_tflops": attention, "tokens_per_device_per_step": flops.tokens_per_device(c)}
  print(json.dumps(out))
  return out


if __name__ == "__main__":
  main()
