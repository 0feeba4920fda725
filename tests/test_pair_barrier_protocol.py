"""Model of the two-CTA GEMM's barrier protocol (lex_gpu_b200/csrc/gemm_fp4_sm100_pair.cuh) under random interleavings.

One cluster: two x producers, two packed-weight producers, 2 x 16 decode warps in four groups (a group owns every
fourth K step), the partner's relay and the MMA warp, with parity waits on barriers that count arrivals exactly as
the kernel's do (`KS` K steps of 64 columns per ring stage: 1, or 2 when the W tiles live in tensor memory).  The model checks what the kernel relies on: no parity wait passes before the phase it stands for
has completed, no W stage is overwritten while its K step is still to be multiplied, and the MMA warp only starts a
K step whose tiles are complete.  It also shows why the barrier rings are at least 4 deep: with a shallower ring a
decode group, which visits the `done` ring every fourth K step, can find the barrier two phases behind the one it
awaits, and the parity test passes early.
"""
import pytest

import random


def run(SX, SW, SR, KB, seed, DNmin, KS=1):
    rnd = random.Random(seed)
    DN = max(SX, SW, DNmin)
    class Bar:
        def __init__(s, count, name): s.count=count; s.pending=count; s.done=0; s.name=name
        def arrive(s):
            s.pending -= 1
            assert s.pending >= 0
            if s.pending == 0: s.pending = s.count; s.done += 1
        def test(s, parity): return (s.done & 1) != parity
    NST = KB // KS                       # stage steps: KS K steps of 64 columns each
    full=[Bar(2+4*KS+1,f"full{j}") for j in range(DN)]
    done=[[Bar(1,f"done{c}_{j}") for j in range(DN)] for c in range(2)]
    wpart=[Bar(4*KS,f"wpart{j}") for j in range(SW)]
    rawf=[[Bar(1,"rawf") for _ in range(SR)] for c in range(2)]
    rawe=[[Bar(16,"rawe") for _ in range(SR)] for c in range(2)]
    mma_done=[-1]      # highest K step whose MMAs completed
    errors=[]
    # ground-truth state for checking
    wslot=[[None]*SW for _ in range(2)]   # which K step's tile is in the slot (per CTA) and complete
    xslot=[[None]*SX for _ in range(2)]
    def wait(bar, parity, truth, what):
        while not bar.test(parity): yield
        if not truth(): errors.append(f"false pass: {what}")
    def xprod(c):
        for kb in range(NST):
            if kb >= SX:
                j=kb-SX
                yield from wait(done[c][j%DN], (j//DN)&1, lambda j=j: mma_done[0]>=j, f"xprod{c} done({j})")
            yield
            xslot[c][kb%SX]=kb
            full[kb%DN].arrive(); 
            if full[kb%DN].done-1 > kb//DN: errors.append(f"early arrive x kb={kb}")
            yield
    def rawprod(c):
        for rb in range(KB//4):
            if rb >= SR:
                yield from wait(rawe[c][rb%SR], ((rb-SR)//SR)&1, lambda: True, "rawe")
            yield
            rawf[c][rb%SR].arrive()
    def dec(c, w):
        q = w>>2
        for kb in range(q, KB, 4):
            rb = kb//4
            yield from wait(rawf[c][rb%SR], (rb//SR)&1, lambda: True, "rawf")
            yield
            rawe[c][rb%SR].arrive()
            for _ in range(rnd.randint(0,6)): yield
            st = kb // KS
            if st >= SW:
                j=st-SW
                yield from wait(done[c][j%DN], (j//DN)&1, lambda j=j: mma_done[0]>=j, f"dec{c}.{w} done({j}) for step={st}")
            yield
            # store
            if wslot[c][st%SW] is not None and wslot[c][st%SW][0] > mma_done[0] and wslot[c][st%SW][0] != st:
                errors.append(f"overwrite of live W slot by step={st} (holds {wslot[c][st%SW]})")
            cur = wslot[c][st%SW]
            wslot[c][st%SW] = (st, (cur[1]+1 if cur and cur[0]==st else 1))
            yield
            if c == 0:
                full[st%DN].arrive()
            else:
                wpart[st%SW].arrive()
    def relay():
        for kb in range(NST):
            yield from wait(wpart[kb%SW], (kb//SW)&1, lambda kb=kb: wslot[1][kb%SW]==(kb,4*KS), f"relay kb={kb}")
            yield
            full[kb%DN].arrive()
    def mma():
        for kb in range(NST):
            yield from wait(full[kb%DN], (kb//DN)&1, lambda kb=kb: wslot[0][kb%SW]==(kb,4*KS) and wslot[1][kb%SW]==(kb,4*KS) and xslot[0][kb%SX]==kb and xslot[1][kb%SX]==kb, f"mma kb={kb}")
            for _ in range(rnd.randint(0,3)): yield
            mma_done[0]=kb
            done[0][kb%DN].arrive(); done[1][kb%DN].arrive()
            yield
    actors=[xprod(0),xprod(1),rawprod(0),rawprod(1),relay(),mma()]+[dec(c,w) for c in range(2) for w in range(16)]
    weights=[rnd.random()+0.05 for _ in actors]
    live=list(range(len(actors)))
    steps=0
    while live and not errors:
        i=rnd.choices(live, [weights[a] for a in live])[0]
        try: next(actors[i])
        except StopIteration: live.remove(i)
        steps+=1
        if steps>3_000_000: errors.append("deadlock/livelock"); break
    return errors


@pytest.mark.parametrize("sx,sw", [(2, 2), (4, 2), (3, 5), (4, 3), (6, 5), (2, 7), (3, 3), (2, 3), (8, 8)])
def test_protocol_is_safe_with_barrier_rings_of_at_least_four(sx, sw):
    for seed in range(6):
        assert run(sx, sw, 2, 24, seed, 4) == []


@pytest.mark.parametrize("sx,sw", [(4, 4), (2, 2), (4, 2), (2, 3), (3, 3)])
def test_protocol_is_safe_with_two_k_steps_per_stage(sx, sw):
    """W tiles in tensor memory: a ring stage holds two K steps, two decode groups fill one stage."""
    for seed in range(6):
        assert run(sx, sw, 2, 24, seed, 4, KS=2) == []


@pytest.mark.parametrize("sx,sw", [(2, 2), (3, 3), (3, 2), (2, 3)])
def test_protocol_is_safe_with_four_k_steps_per_stage(sx, sw):
    """A ring stage holds a whole block of four K steps: all four decode groups fill one stage."""
    for seed in range(6):
        assert run(sx, sw, 2, 24, seed, 4, KS=4) == []


def test_a_shallower_barrier_ring_lets_a_parity_wait_pass_early():
    found = [e for seed in range(12) for e in run(2, 2, 2, 24, seed, 1)]
    assert any(e.startswith("false pass") for e in found)
