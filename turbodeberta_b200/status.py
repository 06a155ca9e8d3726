"""Device status words whose reading has been deferred (no host synchronisation at call time)."""
from __future__ import annotations

import torch


class PendingStatus:
    """Status words of calls made with ``check_status=False`` (no host sync at call time), kept until
    ``check_pending_status()`` reads them.  Nothing is ever dropped: once ``FOLD_AT`` blocks of a device have piled up
    they are folded into one block by an element-wise maximum on that device (a launch, not a synchronisation), so a
    caller that never checks holds a bounded number of small tensors and still sees every report when it does."""
    FOLD_AT = 256

    def __init__(self):
        self._by_dev: dict = {}

    def append(self, status: torch.Tensor) -> None:
        lst = self._by_dev.setdefault(status.device, [])
        lst.append(status)
        if len(lst) >= self.FOLD_AT:
            if status.is_cuda and torch.cuda.is_current_stream_capturing():   # folding would be recorded into the graph
                return
            self._by_dev[status.device] = [torch.stack(lst).amax(dim=0)]

    def drain(self) -> list:
        out = [st for lst in self._by_dev.values() for st in lst]
        self._by_dev.clear()
        return out

    def __len__(self) -> int:
        return sum(len(v) for v in self._by_dev.values())


#: the one queue of the process: attention calls and table projections append, check_pending_status() drains
PENDING = PendingStatus()
