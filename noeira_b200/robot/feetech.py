"""Feetech SCS / STS serial-servo protocol over the native serial port.

Packet: ``FF FF id len instr params… checksum`` with ``len = n_params + 2`` and ``checksum = ~(id + len + instr + Σ params)``.
Status packets carry an error byte in the instruction slot.  ``FeetechBus`` implements ping, read, write and
sync-write of the goal position and the present-position read used by the SO-101 arm
(noeira/robot/ feetech packet codec + bus, so101 arm; serial transport noeira/io/serial/).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

PING, READ, WRITE, SYNC_WRITE = 0x01, 0x02, 0x03, 0x83
ADDR_GOAL_POSITION, ADDR_PRESENT_POSITION, ADDR_TORQUE_ENABLE = 42, 56, 40
BROADCAST = 0xFE


def encode_packet(servo_id: int, instr: int, params: Sequence[int] = ()) -> bytes:
    body = [servo_id & 0xFF, len(params) + 2, instr & 0xFF, *[p & 0xFF for p in params]]
    return bytes([0xFF, 0xFF, *body, (~sum(body)) & 0xFF])


def decode_packet(buf: bytes):
    """→ (servo id, error / instruction byte, params, bytes consumed) or None when no complete valid packet starts ``buf``."""
    i = buf.find(b"\xff\xff")
    if i < 0 or len(buf) < i + 6:
        return None
    sid, ln = buf[i + 2], buf[i + 3]
    end = i + 4 + ln
    if ln < 2 or len(buf) < end:
        return None
    body = buf[i + 2: end - 1]
    if (~sum(body)) & 0xFF != buf[end - 1]:
        raise ValueError("checksum mismatch")
    return sid, buf[i + 4], bytes(buf[i + 5: end - 1]), end


class FeetechBus:
    def __init__(self, port, timeout_ms: int = 50):
        self.port, self.timeout_ms = port, timeout_ms

    def _transact(self, pkt: bytes, expect_reply: bool = True):
        self.port.write(pkt)
        if not expect_reply:
            return None
        buf = b""
        for _ in range(8):
            buf += self.port.read(64, self.timeout_ms)
            r = decode_packet(buf)
            if r is not None:
                return r
        raise TimeoutError("no status packet")

    def ping(self, sid: int) -> bool:
        try:
            r = self._transact(encode_packet(sid, PING))
            return r[0] == sid and r[1] == 0
        except TimeoutError:
            return False

    def read(self, sid: int, addr: int, n: int) -> bytes:
        r = self._transact(encode_packet(sid, READ, [addr, n]))
        if r[1] != 0:
            raise IOError(f"servo {sid} error 0x{r[1]:02x}")
        return r[2]

    def write(self, sid: int, addr: int, data: Sequence[int]):
        r = self._transact(encode_packet(sid, WRITE, [addr, *data]))
        if r[1] != 0:
            raise IOError(f"servo {sid} error 0x{r[1]:02x}")

    def read_position(self, sid: int) -> int:
        b = self.read(sid, ADDR_PRESENT_POSITION, 2)
        return b[0] | (b[1] << 8)

    def sync_write_positions(self, targets: Dict[int, int]):
        params: List[int] = [ADDR_GOAL_POSITION, 2]
        for sid, pos in targets.items():
            params += [sid, pos & 0xFF, (pos >> 8) & 0xFF]
        self._transact(encode_packet(BROADCAST, SYNC_WRITE, params), expect_reply=False)


def ticks_to_radians(ticks: int, centre: int = 2048, ticks_per_rev: int = 4096) -> float:
    import math
    return (ticks - centre) * 2 * math.pi / ticks_per_rev


def radians_to_ticks(rad: float, centre: int = 2048, ticks_per_rev: int = 4096) -> int:
    import math
    return int(round(rad * ticks_per_rev / (2 * math.pi))) + centre
