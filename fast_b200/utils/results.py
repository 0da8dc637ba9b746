"""Result rows appended to a file, one JSON object per line.

The reference's testers append a fixed 16-column text row per experiment to
``../fastalltoall_result/<nodes>n_<test>_<unixtime>.txt`` (amd/test_alltoall.cpp:2064-2090) and its
simulator writes ``benchmark/*.txt`` (simulation/test.cpp:235-263). Here every benchmark prints
its rows as JSON and, when given ``--out``, appends the same rows to a file through this class:
self-describing rows that survive added columns, with the context needed to compare runs.
"""
from __future__ import annotations

import json
import os
import socket
import time
from typing import Iterator, Optional


class ResultLog:
    def __init__(self, path: Optional[str], bench: str, **context):
        self.path, self.bench, self.context = path, bench, context
        if path:
            d = os.path.dirname(os.path.abspath(path))
            os.makedirs(d, exist_ok=True)

    def add(self, row: dict) -> dict:
        """Append one row (no-op without a path); returns the row as written."""
        full = {"bench": self.bench, "unix_time": round(time.time(), 3), "host": socket.gethostname(), **self.context, **row}
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(full) + "\n")
        return full

    @staticmethod
    def read(path: str, bench: Optional[str] = None) -> Iterator[dict]:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                row = json.loads(line)
                if bench is None or row.get("bench") == bench:
                    yield row
