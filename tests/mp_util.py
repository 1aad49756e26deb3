"""Helper for tests that run ranks as child processes: a rank that raises reports its traceback
at once and the parent stops waiting as soon as any child has died."""
import queue as _queue
import socket
import traceback

import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(fn, rank, world, port, args, q):
    try:
        fn(rank, world, port, *args, q)
    except BaseException:
        q.put(("__error__", rank, traceback.format_exc()))
        raise


def run_ranks(fn, world: int, args=(), results: int = 1, timeout: float = 240.0):
    """Start ``fn(rank, world, port, *args, queue)`` on ``world`` processes, collect ``results``
    queue items, join.  Raises with the child's traceback if one fails.  Children should put
    plain Python / numpy data (tensors travel as file descriptors and are lost if the child exits
    first)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    out, waited = [], 0.0
    try:
        while len(out) < results:
            try:
                item = q.get(timeout=1.0)
            except _queue.Empty:
                waited += 1.0
                dead = [p for p in procs if p.exitcode not in (None, 0)]
                if dead:
                    raise RuntimeError(f"a rank exited with code {dead[0].exitcode} before reporting")
                if waited > timeout:
                    raise TimeoutError(f"no result after {timeout} s")
                continue
            if isinstance(item, tuple) and item and item[0] == "__error__":
                raise RuntimeError(f"rank {item[1]} failed:\n{item[2]}")
            out.append(item)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    return out
