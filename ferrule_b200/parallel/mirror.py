"""Lock-step command mirror for one model replica spread over several ranks (tensor / pipeline parallel serving).

Only the leader rank (0) talks to clients.  Every rank owns a full `Engine` over its shard of the model; the engines
stay in step because they are deterministic functions of the same command sequence (submissions, cancellations)
and of the tokens the model produced, which are bit-equal on every rank (the fused all-reduces sum in one fixed
order).  Per tick the leader publishes the commands it applied and the fact that it is about to step; followers
apply the same commands and step.  The host transport is a CPU (gloo) process group: one 16-byte header
broadcast per tick, a second broadcast only when commands are attached.

The reference serves one GPU per worker (crates/ferrule-server/src/worker.rs:290-520: one thread owns the
engine, commands arrive over a bounded channel); this is that worker's command stream replayed on the other
ranks of the replica.
"""
from __future__ import annotations

import pickle
from typing import Any, Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

TICK, SHUTDOWN = 0, 1


class CommandMirror:
    def __init__(self, rank: int, world: int, group=None, leader: int = 0):
        self.rank, self.world, self.group, self.leader = rank, world, group, leader
        self.ticks = 0
        self.bytes_sent = 0

    @property
    def is_leader(self) -> bool:
        return self.rank == self.leader

    # ---------------------------------------------------------------- leader
    def publish(self, commands: List[Tuple], kind: int = TICK) -> None:
        payload = pickle.dumps(commands, protocol=pickle.HIGHEST_PROTOCOL) if commands else b""
        head = torch.tensor([kind, len(payload)], dtype=torch.int64)
        dist.broadcast(head, src=self.leader, group=self.group)
        if payload:
            dist.broadcast(torch.frombuffer(bytearray(payload), dtype=torch.uint8), src=self.leader, group=self.group)
        self.ticks += 1
        self.bytes_sent += 16 + len(payload)

    def shutdown(self) -> None:
        self.publish([], SHUTDOWN)

    # ---------------------------------------------------------------- follower
    def receive(self) -> Tuple[int, List[Tuple]]:
        head = torch.zeros(2, dtype=torch.int64)
        dist.broadcast(head, src=self.leader, group=self.group)
        kind, n = int(head[0]), int(head[1])
        cmds: List[Tuple] = []
        if n:
            buf = torch.empty(n, dtype=torch.uint8)
            dist.broadcast(buf, src=self.leader, group=self.group)
            cmds = pickle.loads(buf.numpy().tobytes())
        self.ticks += 1
        return kind, cmds


def apply_command(engine, cmd: Tuple) -> None:
    """A mirrored command on a follower's engine: ("submit", GenerateRequest fields...) or ("cancel", request id)."""
    from ..runtime.session import GenerateRequest
    if cmd[0] == "submit":
        _, rid, ids, max_tokens, stop, ignore_eos, session_id = cmd
        engine.submit(GenerateRequest(rid, list(ids), max_new_tokens=max_tokens, stop=list(stop), ignore_eos=ignore_eos,
                                      session_id=session_id, retain_session=session_id is not None))
    elif cmd[0] == "cancel":
        engine.cancel_request(cmd[1])
    else:
        raise ValueError(f"unknown mirrored command {cmd[0]!r}")


def follower_loop(engine, mirror: CommandMirror, emit: Optional[Callable[[Any], None]] = None) -> int:
    """Run a follower rank until the leader shuts down; returns the number of engine steps taken."""
    sink = emit or (lambda ev: None)
    steps = 0
    while True:
        kind, cmds = mirror.receive()
        if kind == SHUTDOWN:
            break
        for c in cmds:
            apply_command(engine, c)
        engine.step(sink)
        steps += 1
    for _ in range(1000):
        if engine.shutdown():
            break
    return steps
