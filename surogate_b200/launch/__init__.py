"""Launchers: start a training run on this machine, on an SSH host, on cloud GPUs through dstack, or in a Modal sandbox, with
every run in a directory of its own and its metrics feed mirrored back to this machine, so ``surogate monitor`` follows a remote
run exactly as it follows a local one.

  runs.py        one directory per run (feed, config, log, meta, output), run history
  records.py     which lines of a stream are feed records
  stream.py      pump a child's stdout into feed + log; mirror a remote file with reconnects
  providers.py   saved compute targets (non-secret metadata only)
  configs.py     a training config from a handful of launch fields; monitoring / resume overlays
  fit.py         rough memory estimate of a run and whether it fits a GPU
  local.py ssh.py dstack.py modal.py     the four targets
  artifacts.py   bring a finished run's outputs back

Parity: jackalope/src/{runs,records,feed-pipe,providers,launch,ssh,dstack,modal,artifacts}.ts (a TypeScript dashboard in the
reference; here a Python package behind ``surogate launch`` and ``surogate monitor``).
"""
from .configs import LaunchFields, build_config, monitoring_overlay, resume_overlay  # noqa: F401
from .fit import estimate_run_memory_gb, fit_verdict, params_billions  # noqa: F401
from .providers import ProviderRecord, ProviderStore, provider_id  # noqa: F401
from .runs import RunDir, list_runs, new_run  # noqa: F401
