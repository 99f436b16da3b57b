"""Randomised-schedule model of the barrier protocol of the two-tile attention forward (``attn_fwd2_kernel`` in
``csrc/attention_tcgen05.cu``): one MMA / TMA issuing thread and two softmax groups that share each K and V block.

The model follows the kernel's order of waits, loads, MMAs and commits one for one (mbarrier parities included: a
wait succeeds when the barrier's completed-phase count has the other parity) and runs it under random latencies
of loads, MMAs and softmax work.  It checks what the kernel's correctness rests on: no deadlock, no K or V block
overwritten before the MMAs that read it have completed, no S or O accumulator overwritten before its softmax
group has read it, no P tile overwritten before the P·V product that reads it has completed, and every MMA
issued with the operands of the block it belongs to.  A protocol change in the kernel has to be made here too.
"""
import random

import pytest


class Bar:
    def __init__(self, need=1): self.need, self.arrived, self.completions = need, 0, 0
    def arrive(self):
        self.arrived += 1
        if self.arrived == self.need: self.arrived = 0; self.completions += 1
    def test(self, parity): return (self.completions & 1) != parity

def run(nkb0, nkb1, seed):
    rnd = random.Random(seed)
    nkb = max(nkb0, nkb1)
    nk = [nkb0, nkb1]
    B = {n: Bar() for n in ("q_full","k_full","k_empty","v_full","v_empty")}
    for g in range(2):
        B[f"s_full{g}"]=Bar(); B[f"p_ready{g}"]=Bar(1); B[f"pv_full{g}"]=Bar()   # softmax group modelled as one agent
    pending=[]   # (time, action)
    now=[0.0]
    mma_busy_until=[0.0]
    state={"k_in_smem":-1,"v_in_smem":-1,"k_loading":None,"v_loading":None,
           "S":[-1,-1],"S_read":[-1,-1],"O":[-1,-1],"O_read":[-1,-1],"P":[-1,-1],
           "s_done":[-1,-1],"pv_done":[-1,-1], "s_inflight":[None,None], "pv_inflight":[None,None]}
    errors=[]
    def at(t,f): pending.append((t,rnd.random(),f))
    def load(kind,kb):
        # hazard: previous block must have been fully consumed by the MMAs that read it
        if kind=="k":
            for g in range(2):
                if kb-1 < nk[g] and kb-1>=0 and state["s_done"][g] < kb-1: errors.append(f"K overwritten before S{g}({kb-1}) done")
        else:
            for g in range(2):
                if kb-1 < nk[g] and kb-1>=0 and state["pv_done"][g] < kb-1: errors.append(f"V overwritten before PV{g}({kb-1}) done")
        def done():
            state[f"{kind}_in_smem"]=kb; B[f"{kind}_full"].arrive()
        at(now[0]+rnd.uniform(0.5,3.0), done)
    def issue_mma(kind,g,kb):
        start=max(now[0], mma_busy_until[0]); end=start+rnd.uniform(0.2,1.0); mma_busy_until[0]=end
        if kind=="s":
            if state["k_in_smem"]!=kb: errors.append(f"S{g}({kb}) issued with K block {state['k_in_smem']}")
            if state["S_read"][g] < kb-1: errors.append(f"S{g}({kb}) overwrites unread S({kb-1})")
            def done(): state["S"][g]=kb; state["s_done"][g]=kb
        else:
            if state["v_in_smem"]!=kb: errors.append(f"PV{g}({kb}) issued with V block {state['v_in_smem']}")
            if state["P"][g]!=kb: errors.append(f"PV{g}({kb}) issued with P block {state['P'][g]}")
            if state["O_read"][g] < kb-1: errors.append(f"PV{g}({kb}) overwrites unread O({kb-1})")
            def done(): state["O"][g]=kb; state["pv_done"][g]=kb
        at(end, done)
        return end
    def commit(bar):
        t=mma_busy_until[0]   # arrives when everything issued so far has completed
        at(max(t,now[0])+1e-6, lambda: B[bar].arrive())

    def mma_thread():
        if nkb>0:
            load("k",0); load("v",0)
            yield ("wait","k_full",0)   # q_full folded in
            if 0<nk[0]: issue_mma("s",0,0); commit("s_full0")
            if 0<nk[1]: issue_mma("s",1,0); commit("s_full1")
            commit("k_empty")
        for kb in range(nkb):
            ph=kb&1; more=kb+1<nkb
            if more:
                yield ("wait","k_empty",ph); load("k",kb+1)
            yield ("wait","v_full",ph)
            if kb<nk[0]:
                yield ("wait","p_ready0",ph); issue_mma("pv",0,kb); commit("pv_full0")
            if more:
                yield ("wait","k_full",ph^1)
                if kb+1<nk[0]: issue_mma("s",0,kb+1); commit("s_full0")
            if kb<nk[1]:
                yield ("wait","p_ready1",ph); issue_mma("pv",1,kb); commit("pv_full1")
            commit("v_empty")
            if more:
                if kb+1<nk[1]: issue_mma("s",1,kb+1); commit("s_full1")
                commit("k_empty")
                yield ("wait","v_empty",ph); load("v",kb+1)
    def softmax(g):
        for kb in range(nk[g]):
            yield ("wait",f"s_full{g}",kb&1)
            if state["S"][g]!=kb: errors.append(f"softmax{g} reads S block {state['S'][g]} expecting {kb}")
            yield ("sleep", rnd.uniform(0.3,2.5))
            state["S_read"][g]=kb
            if kb>0 and state["pv_done"][g] < kb-1: errors.append(f"softmax{g} overwrites P({kb-1}) before PV done")
            state["P"][g]=kb
            B[f"p_ready{g}"].arrive()
            yield ("wait",f"pv_full{g}",kb&1)
            if state["O"][g]!=kb: errors.append(f"softmax{g} reads O block {state['O'][g]} expecting {kb}")
            yield ("sleep", rnd.uniform(0.1,0.8))
            state["O_read"][g]=kb
    agents={"mma":mma_thread(),"sm0":softmax(0),"sm1":softmax(1)}
    waiting={}; sleeping={}
    def step(name):
        try:
            req=next(agents[name])
        except StopIteration:
            del agents[name]; return
        if req[0]=="wait": waiting[name]=(req[1],req[2])
        else: sleeping[name]=now[0]+req[1]
    for n in list(agents): step(n)
    guard=0
    while agents:
        guard+=1
        if guard>100000: return ["livelock"]
        progressed=False
        for n,(bar,par) in list(waiting.items()):
            if B[bar].test(par):
                del waiting[n]; step(n); progressed=True
        for n,t in list(sleeping.items()):
            if t<=now[0]:
                del sleeping[n]; step(n); progressed=True
        if progressed: continue
        times=[t for t,_,_ in pending]+list(sleeping.values())
        if not times:
            return errors+[f"DEADLOCK waiting={waiting} completions={{k:v.completions for k,v in B.items()}}".replace("{k:v.completions for k,v in B.items()}", str({k:v.completions for k,v in B.items()}))]
        tmin=min(times); now[0]=tmin
        due=[p for p in pending if p[0]<=tmin]; due.sort()
        for p in due:
            pending.remove(p); p[2]()
    return errors


@pytest.mark.parametrize("nkb0,nkb1", [(1, 1), (2, 2), (3, 3), (8, 8), (1, 2), (3, 4), (7, 8), (2, 0), (5, 0), (1, 0),
                                       (4, 5)])
def test_two_tile_attention_protocol_has_no_deadlock_or_hazard(nkb0, nkb1):
    for seed in range(60):
        assert run(nkb0, nkb1, seed) == [], (nkb0, nkb1, seed)


def test_the_model_notices_a_missing_wait():
    """The checks are live: dropping the wait that protects the K buffer is reported."""
    import types
    source = open(__file__).read().replace('yield ("wait","k_empty",ph); load("k",kb+1)', 'load("k",kb+1)')
    broken = types.ModuleType("broken_protocol")
    exec(compile(source, "broken_protocol", "exec"), broken.__dict__)
    assert any(broken.run(3, 4, seed) for seed in range(20))
