"""Single-slot "latest frame wins" mailbox between the decode loop and a consumer
(src/viz/transport.rs:15-77): sending never blocks and overwrites an unread frame; draining takes
the frame and leaves the slot empty."""
from __future__ import annotations

import threading
from typing import Any, Optional, Tuple


class _Slot:
    def __init__(self):
        self.lock = threading.Lock()
        self.frame: Optional[Any] = None


class VizSender:
    def __init__(self, slot: _Slot):
        self._slot = slot

    def try_send(self, frame) -> None:
        if self._slot.lock.acquire(blocking=False):
            try:
                self._slot.frame = frame
            finally:
                self._slot.lock.release()


class VizReceiver:
    def __init__(self, slot: _Slot):
        self._slot = slot

    def drain_latest(self):
        with self._slot.lock:
            f, self._slot.frame = self._slot.frame, None
            return f


def channel() -> Tuple[VizSender, VizReceiver]:
    s = _Slot()
    return VizSender(s), VizReceiver(s)
