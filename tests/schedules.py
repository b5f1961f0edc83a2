"""Ways of cutting the same requests into steps.  Each function returns a list of steps
in the trace-replay format: {"step", "entries": [{"id", "tokens", "want"}], "end"}.
Every step asks for the logits of all its tokens, so each schedule yields the logits of
every position of every request, to be compared with the plain implementation.
"""
import random
from typing import Dict, List, Sequence


def _entry(rid, tokens):
    return {"id": rid, "tokens": list(tokens), "want": list(range(len(tokens)))}


def whole(requests: Dict[str, Sequence[int]]) -> List[dict]:
    """Each request alone and whole, one step per request."""
    steps = []
    for rid, ids in requests.items():
        steps.append({"step": len(steps), "entries": [_entry(rid, ids)], "end": [rid]})
    return steps


def tail_decode(requests: Dict[str, Sequence[int]], tail: int = 32) -> List[dict]:
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": len(steps), "entries": [_entry(rid, ids[:head])], "end": []})
        for i in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [_entry(rid, ids[i:i + 1])],
                          "end": [rid] if i == len(ids) - 1 else []})
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: Dict[str, Sequence[int]], sizes=(7, 2, 19, 3, 2, 16, 5, 33, 2)) -> List[dict]:
    """Portions of changing size, down to two tokens, each request alone."""
    steps = []
    for rid, ids in requests.items():
        i, k = 0, 0
        while i < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - i)
            k += 1
            steps.append({"step": len(steps), "entries": [_entry(rid, ids[i:i + n])],
                          "end": [rid] if i + n == len(ids) else []})
            i += n
    return steps


def mixed(requests: Dict[str, Sequence[int]], seed: int = 0, max_live: int = 4,
          decode_tail: int = 8) -> List[dict]:
    """Up to `max_live` live requests: portions of some beside single tokens of others.
    A request runs its prompt in random portions, then its last `decode_tail` tokens one
    at a time; some steps leave a live request out.  Requests start as others end, so
    freed pages are handed out again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}          # rid -> [ids, done]
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = [list(ids), 0]
        entries, end = [], []
        for rid, (ids, done) in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                      # sits this step out
            left = len(ids) - done
            if left <= decode_tail:
                n = 1
            else:
                n = min(left - decode_tail, rng.choice([2, 3, 5, 8, 13, 21, 40]))
            entries.append(_entry(rid, ids[done:done + n]))
            live[rid][1] = done + n
            if done + n == len(ids):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def tokens_held(steps: List[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to `round_to`."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def replay(runner, steps: List[dict]):
    """Run steps on a ModelRunner; {(id, position): logits row (cpu float32)}."""
    import torch
    from rvllm_b200.engine import StepEntry
    out, pos = {}, {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not runner.cache.has(e["id"]):
                runner.add_request(e["id"])
                pos[e["id"]] = 0
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = runner.step(entries).to("cpu", torch.float32)
        k = 0
        for e in s["entries"]:
            for w in e["want"]:
                out[(e["id"], pos[e["id"]] + w)] = logits[k]
                k += 1
            pos[e["id"]] += len(e["tokens"])
        for rid in s["end"]:
            runner.end_request(rid)
        runner.cache.check()
    return out
