"""Tombstones: a job can be stopped from outside the scheduler by creating a file.  A watcher
thread polls for ``scancel_<jobid>``-style files in the user's tombstone directory and, when one
appears, cancels (or requeues) the job through ``scancel`` / ``scontrol`` (reference:
metaseq/launcher/tombyard.py:39-112)."""
from __future__ import annotations

import os
import subprocess
import threading
import time
from pathlib import Path
from typing import Callable, Dict, Optional


def tombstones(job_id: str, base_dir: str) -> Dict[str, str]:
    base = Path(base_dir)
    return {
        "scancel": str(base / f"scancel_{job_id}"),
        "requeuehold": str(base / f"requeuehold_{job_id}"),
        "release": str(base / f"release_{job_id}"),
    }


def _default_actions(job_id: str) -> Dict[str, Callable[[], None]]:
    return {
        "scancel": lambda: subprocess.run(["scancel", job_id]),
        "requeuehold": lambda: subprocess.run(["scontrol", "requeuehold", job_id]),
        "release": lambda: subprocess.run(["scontrol", "release", job_id]),
    }


def tombstones_procedure(job_id: str, base_dir: str, period: float = 60.0, dirstones=None,
                         actions: Optional[Dict[str, Callable[[], None]]] = None, stop_event=None, max_polls=None):
    """Polls until a tombstone shows up, runs its action and removes the file."""
    stones = tombstones(job_id, base_dir)
    actions = actions or _default_actions(job_id)
    polls = 0
    while stop_event is None or not stop_event.is_set():
        for kind, path in stones.items():
            if os.path.exists(path):
                print(f"tombyard: found {path}; running '{kind}' for job {job_id}", flush=True)
                actions[kind]()
                try:
                    os.remove(path)
                except OSError:
                    pass
                if kind == "scancel":
                    return kind
        polls += 1
        if max_polls is not None and polls >= max_polls:
            return None
        time.sleep(period)
    return None


def tombyard(job_id: Optional[str] = None, base_dir: Optional[str] = None, period: float = 60.0) -> Optional[threading.Thread]:
    """Starts the watcher thread for the current SLURM job (no-op outside SLURM)."""
    job_id = job_id or os.environ.get("SLURM_JOB_ID")
    if job_id is None:
        return None
    base_dir = base_dir or os.path.join(os.path.expanduser("~"), "tombstones")
    os.makedirs(base_dir, exist_ok=True)
    t = threading.Thread(target=tombstones_procedure, args=(job_id, base_dir, period), daemon=True)
    t.start()
    return t
