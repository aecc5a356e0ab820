"""Configuration loader: default table -> YAML chain -> model catalog -> CLI -> environment.

Behavioural contract (same as MaxText's `pyconfig.initialize`, src/maxtext/configs/pyconfig.py:403-586):

* ``argv[1]`` is a YAML path, the remaining arguments are ``key=value`` overrides;
* a YAML file may name a parent with ``base_config:`` (resolved next to the file, then in the
  packaged ``configs/`` directory); parents are applied first;
* ``model_name=<x>`` merges ``configs/models/<x>.yml``; those architecture constants beat the YAML
  chain, and a CLI override of one of them is an error unless ``override_model_config=true``;
* ``M_<KEY>`` environment variables override like CLI arguments; setting the same key on the CLI
  and in the environment is an error (pyconfig.py:128);
* unknown keys are errors;
* ``logical_axis_rules`` given by the user are merged by logical-axis name into the default table
  unless ``override_logical_axis_rules=true`` (pyconfig.py:166-185);
* derived values are filled in by :func:`maxtext_b200.config.types.derive_and_validate`;
* the result (:class:`HyperParameters`) is read-only.

Unlike the reference, the defaults do not live in a YAML file: they are the typed table in
``defaults.py`` and ``configs/base.yml`` is an (almost) empty override layer. Nothing here boots a
distributed runtime; that is the job of ``parallel.mesh.init_distributed``.
"""
from __future__ import annotations

import copy
import os
import sys
from typing import Any

import yaml

from . import defaults as _defaults
from . import types as _types

CONFIG_ROOT = os.path.normpath(os.path.join(os.path.dirname(__file__), "..", "configs"))
_ENV_PREFIX = "M_"


class ConfigError(ValueError):
  pass


def _find_yaml(path: str, relative_to: str | None = None) -> str:
  cands = [path]
  if relative_to:
    cands.append(os.path.join(relative_to, path))
  cands.append(os.path.join(CONFIG_ROOT, path))
  cands.append(os.path.join(CONFIG_ROOT, os.path.basename(path)))
  # the reference spells its paths "src/maxtext/configs/<x>"; accept them
  marker = "configs/"
  if marker in path:
    cands.append(os.path.join(CONFIG_ROOT, path.split(marker, 1)[1]))
  for c in cands:
    if os.path.isfile(c):
      return c
  raise ConfigError(f"config file not found: {path} (tried {cands})")


def load_yaml_chain(path: str) -> dict:
  """Return the merged dict of a YAML file and its ``base_config`` ancestors (ancestors first)."""
  real = _find_yaml(path)
  seen = set()
  layers = []
  while True:
    if real in seen:
      raise ConfigError(f"base_config cycle at {real}")
    seen.add(real)
    with open(real, "r", encoding="utf-8") as fh:
      data = yaml.safe_load(fh) or {}
    if not isinstance(data, dict):
      raise ConfigError(f"{real} does not hold a mapping")
    parent = data.pop("base_config", None)
    layers.append(data)
    if not parent:
      break
    real = _find_yaml(parent, os.path.dirname(real))
  out: dict = {}
  for layer in reversed(layers):
    out.update(layer)
  return out


def _coerce(key: str, value: Any, default: Any) -> Any:
  """Bring a user value to the type of the default for that key."""
  if isinstance(value, str) and value in ("None", "none", "null") and not isinstance(default, str):
    return None
  if default is None or value is None:
    return value
  if isinstance(default, bool):
    if isinstance(value, bool):
      return value
    if isinstance(value, (int, float)):
      return bool(value)
    if isinstance(value, str):
      low = value.strip().lower()
      if low in ("true", "1", "yes", "y", "t"):
        return True
      if low in ("false", "0", "no", "n", "f", ""):
        return False
    raise ConfigError(f"{key}: cannot read {value!r} as a boolean")
  if isinstance(default, int) and not isinstance(default, bool):
    if isinstance(value, bool):
      return int(value)
    if isinstance(value, int):
      return value
    if isinstance(value, float):
      if value != int(value):
        return value  # e.g. per-device batch given as a fraction for an int default: keep
      return int(value)
    if isinstance(value, str):
      try:
        return int(value.replace("_", ""))
      except ValueError:
        try:
          return float(value)
        except ValueError as e:
          raise ConfigError(f"{key}: cannot read {value!r} as an integer") from e
  if isinstance(default, float):
    if isinstance(value, (int, float)) and not isinstance(value, bool):
      return float(value)
    if isinstance(value, str):
      try:
        return float(value)
      except ValueError as e:
        raise ConfigError(f"{key}: cannot read {value!r} as a float") from e
  if isinstance(default, str):
    if isinstance(value, (list, dict)):
      return value
    return str(value)
  if isinstance(default, (list, tuple)) and isinstance(value, str):
    parsed = yaml.safe_load(value)
    if isinstance(parsed, (list, tuple)):
      return list(parsed)
    return [parsed]
  return value


def parse_cli(args: list[str]) -> dict:
  out = {}
  for a in args:
    if "=" not in a:
      raise ConfigError(f"expected key=value, got {a!r}")
    k, v = a.split("=", 1)
    k = k.strip()
    if k in out:
      raise ConfigError(f"key {k} given twice on the command line")
    try:
      out[k] = yaml.safe_load(v) if v != "" else ""
    except yaml.YAMLError:
      out[k] = v
  return out


def merge_logical_axis_rules(base_rules: list, user_rules: list) -> list:
  """User rules replace every default rule of the same logical name, in place of the first one.

  New logical names are appended. Order of untouched rules is kept because resolution is
  first-match.
  """
  user_by_name: dict[str, list] = {}
  order: list[str] = []
  for name, axes in user_rules:
    if name not in user_by_name:
      user_by_name[name] = []
      order.append(name)
    user_by_name[name].append([name, axes])
  out, done = [], set()
  for name, axes in base_rules:
    if name in user_by_name:
      if name not in done:
        out.extend(user_by_name[name])
        done.add(name)
      continue
    out.append([name, axes])
  for name in order:
    if name not in done:
      out.extend(user_by_name[name])
  return out


class HyperParameters:
  """Read-only attribute view over the final key table."""

  __slots__ = ("_keys",)

  def __init__(self, keys: dict):
    object.__setattr__(self, "_keys", keys)

  def __getattr__(self, name: str):
    keys = object.__getattribute__(self, "_keys")
    try:
      return keys[name]
    except KeyError:
      raise AttributeError(f"config has no key {name!r}") from None

  def __setattr__(self, name, value):
    raise AttributeError("configuration is read-only; build a new one with pyconfig.initialize")

  def __contains__(self, name):
    return name in self._keys

  def get_keys(self) -> dict:
    return copy.deepcopy(self._keys)

  def replace(self, **kw) -> "HyperParameters":
    """A new config with some raw keys changed and derived values recomputed."""
    raw = {k: v for k, v in self._keys.items() if k in _defaults.DEFAULTS}
    raw.update(kw)
    return HyperParameters(_types.derive_and_validate(raw, num_devices=kw.pop("_num_devices", self._keys["num_target_devices"])))

  def __repr__(self):
    return f"HyperParameters({len(self._keys)} keys, model={self._keys.get('model_name')})"


def initialize(argv: list[str] | None = None, num_devices: int | None = None, **kwargs) -> HyperParameters:
  """Build the configuration.

  ``argv`` follows the CLI shape ``[prog, yaml_path, key=value...]``; ``kwargs`` are overrides with
  CLI priority. ``num_devices`` fixes the device count used for batch-size and mesh derivation
  (defaults to WORLD_SIZE, else the visible CUDA devices of this process group, else 1).
  """
  argv = list(argv) if argv is not None else list(sys.argv)
  table = copy.deepcopy(_defaults.DEFAULTS)
  yaml_path = None
  cli_args = []
  for a in argv[1:]:
    if yaml_path is None and "=" not in a:
      yaml_path = a
    else:
      cli_args.append(a)
  file_keys = load_yaml_chain(yaml_path) if yaml_path else {}
  cli = parse_cli(cli_args)
  for k, v in kwargs.items():
    if k in cli:
      raise ConfigError(f"key {k} given both as argument and on the command line")
    cli[k] = v

  env = {}
  for name, v in os.environ.items():
    if name.startswith(_ENV_PREFIX):
      key = name[len(_ENV_PREFIX):].lower()
      if key in table:
        if key in cli:
          raise ConfigError(f"key {key} is set on the command line and by environment variable {name}")
        try:
          env[key] = yaml.safe_load(v)
        except yaml.YAMLError:
          env[key] = v

  def check_known(src: dict, where: str):
    unknown = [k for k in src if k not in table]
    if unknown:
      raise ConfigError(f"unknown configuration key(s) {unknown} in {where}")

  check_known(file_keys, yaml_path or "<yaml>")
  check_known(cli, "command line")

  user_rules = None
  for src in (file_keys, env, cli):
    for k, v in src.items():
      if k == "logical_axis_rules":
        user_rules = v if user_rules is None else merge_logical_axis_rules(user_rules, v)
        continue
      table[k] = _coerce(k, v, _defaults.DEFAULTS[k])

  # custom mesh + rule set replaces mesh_axes / rules / data_sharding wholesale
  cmr = table.get("custom_mesh_and_rule") or ""
  if cmr:
    over = load_yaml_chain(os.path.join("custom_mesh_and_rule", f"{cmr}.yml"))
    for k, v in over.items():
      table[k] = v

  if user_rules is not None:
    if table.get("override_logical_axis_rules"):
      table["logical_axis_rules"] = [list(r) for r in user_rules]
    else:
      table["logical_axis_rules"] = merge_logical_axis_rules(table["logical_axis_rules"], user_rules)

  # model catalog
  model_name = table.get("model_name", "default")
  if model_name and model_name != "default":
    mpath = os.path.join(CONFIG_ROOT, "models", f"{model_name}.yml")
    if not os.path.isfile(mpath):
      raise ConfigError(f"model_name={model_name}: no such catalog entry {mpath}")
    with open(mpath, "r", encoding="utf-8") as fh:
      mkeys = yaml.safe_load(fh) or {}
    check_known(mkeys, mpath)
    explicit = set(cli) | set(env)
    for k, v in mkeys.items():
      if k in explicit:
        if not table.get("override_model_config"):
          raise ConfigError(
              f"{k} is fixed by model_name={model_name}; pass override_model_config=true to change it")
        continue
      table[k] = _coerce(k, v, _defaults.DEFAULTS[k])

  if num_devices is None:
    num_devices = _types.detect_num_devices(table)
  final = _types.derive_and_validate(table, num_devices=num_devices)
  hp = HyperParameters(final)
  if final.get("log_config") and os.environ.get("MAXTEXT_B200_QUIET", "") == "" and int(os.environ.get("RANK", "0")) == 0:
    from ..utils import max_logging
    for k in sorted(final):
      max_logging.debug(f"Config param {k}: {final[k]}")
  return hp


# kept for callers that do `pyconfig.initialize_pydantic`-style access in the reference
initialize_config = initialize
