"""Start a multi-node job from one machine over ssh (the role of tools/orchestration/multihost_runner.py, which drives TPU VMs
through gcloud; here the nodes are GPU hosts reachable by ssh).

  python -m maxtext_b200.orchestration.multihost_runner --hosts node0,node1 --gpus-per-node 8 [--workdir /path/to/repo] \\
      [--port 29500] [--env NCCL_DEBUG=WARN] [--dry-run] -- python -m maxtext.train maxtext_b200/configs/base.yml model_name=llama3-8b ...

Every host runs `orchestration/gpu_multi_process_run.sh` with NNODES / NODE_RANK / coordinator variables set, which in turn
starts one rank per GPU. Output of every host is prefixed with its name; the first failing host ends the job (the others are
asked to stop through their ssh sessions). `--dry-run` prints the per-host command lines instead of running them.
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
import threading


def host_commands(hosts: list[str], gpus_per_node: int, command: list[str], workdir: str, port: int = 29500, env: dict | None = None,
                  ssh_options: str = "-o BatchMode=yes -o StrictHostKeyChecking=accept-new") -> list[list[str]]:
  """One ssh argv per host. Node 0 is the coordinator."""
  if not hosts:
    raise ValueError("no hosts given")
  script = os.path.join(workdir, "maxtext_b200", "orchestration", "gpu_multi_process_run.sh")
  out = []
  for rank, host in enumerate(hosts):
    variables = {"NNODES": len(hosts), "NODE_RANK": rank, "JAX_COORDINATOR_ADDRESS": hosts[0], "JAX_COORDINATOR_PORT": port,
                 "GPUS_PER_NODE": gpus_per_node, "COMMAND": " ".join(shlex.quote(c) for c in command), **(env or {})}
    assigns = " ".join(f"{k}={shlex.quote(str(v))}" for k, v in variables.items())
    remote = f"cd {shlex.quote(workdir)} && {assigns} bash {shlex.quote(script)}"
    out.append(["ssh", *shlex.split(ssh_options), host, remote])
  return out


def _pump(name, stream, sink):
  for line in iter(stream.readline, ""):
    sink.write(f"[{name}] {line}")
    sink.flush()


def run(hosts, gpus_per_node, command, workdir, port=29500, env=None, runner=subprocess.Popen, sink=sys.stdout) -> int:
  procs = []
  for host, argv in zip(hosts, host_commands(hosts, gpus_per_node, command, workdir, port, env)):
    p = runner(argv, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    t = threading.Thread(target=_pump, args=(host, p.stdout, sink), daemon=True)
    t.start()
    procs.append((host, p, t))
  rc = 0
  pending = list(procs)
  while pending:
    for item in list(pending):
      host, p, t = item
      code = p.poll()
      if code is None:
        continue
      pending.remove(item)
      t.join(timeout=5)
      if code != 0 and rc == 0:
        rc = code
        sink.write(f"[{host}] exited with {code}; stopping the other hosts\n")
        for _, q, _ in pending:
          q.terminate()                     # the ssh session this runner started; the remote shell gets SIGHUP
    if pending:
      try:
        pending[0][1].wait(timeout=0.2)
      except subprocess.TimeoutExpired:
        pass
  return rc


def main(argv=None):
  argv = list(sys.argv[1:] if argv is None else argv)
  if "--" not in argv:
    print(__doc__)
    return 2
  cut = argv.index("--")
  ap = argparse.ArgumentParser()
  ap.add_argument("--hosts", required=True, help="comma-separated host names, or @file with one host per line")
  ap.add_argument("--gpus-per-node", type=int, default=8)
  ap.add_argument("--workdir", default=os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
  ap.add_argument("--port", type=int, default=29500)
  ap.add_argument("--env", action="append", default=[])
  ap.add_argument("--dry-run", action="store_true")
  a = ap.parse_args(argv[:cut])
  command = argv[cut + 1:]
  hosts = [h.strip() for h in (open(a.hosts[1:]).read().split() if a.hosts.startswith("@") else a.hosts.split(",")) if h.strip()]
  env = dict(e.split("=", 1) for e in a.env)
  if a.dry_run:
    for c in host_commands(hosts, a.gpus_per_node, command, a.workdir, a.port, env):
      print(" ".join(shlex.quote(x) for x in c))
    return 0
  return run(hosts, a.gpus_per_node, command, a.workdir, a.port, env)


if __name__ == "__main__":
  sys.exit(main())
