"""The fused directory kernels replay the planner traces recorded from the reference (tests/golden/dir_*.npz): every
output of every call and the directory state after every call must equal the reference's C++ directory."""
import numpy as np
import pytest
import torch

from test_oracle_golden import run_dir_trace, crc_check

pytestmark = pytest.mark.gpu


class GpuDirectory:
    def __init__(self, O, st, pv, dev):
        from elara_b200.ops import dir_ext
        self.O, self.dx, self.dev = O, dir_ext(), dev
        self.t = {k: torch.from_numpy(np.ascontiguousarray(st[k], O.DIR_DTYPES[k]).copy()).to(dev) for k in O.DIR_FIELDS}
        self.stv = [self.t[k] for k in O.DIR_FIELDS]
        self.pv = [pv[k] for k in ('R', 'K', 'Lcap', 'n0', 'Cdyn', 'MAT', 'trash', 'evl')]

    def _d(self, a, dt=torch.int64):
        return torch.from_numpy(np.ascontiguousarray(a)).to(self.dev).to(dt)

    def dir_a(self, hs, L_row, L_cnt, ev_slot, s):
        o = self.dx.elara_dir_a(self.stv, self.pv, self._d(hs), self._d(L_row), self._d(L_cnt, torch.int32), self._d(ev_slot), s)
        names = ('L_steps', 'L_ids', 'hrec_dyn', 'hrec_j', 'ev_row', 'rep', 'evl_ids', 'evf_slots', 'ev_dyn')
        assert o[5].dtype == torch.bool and o[0].dtype == torch.int32 and o[6].dtype == torch.int64
        return {k: v.cpu().numpy() for k, v in zip(names, o)}

    def admit(self, adm_rows, adm_slots, lazy_n, s):
        self.dx.admit(self.stv, self.pv, self._d(adm_rows), self._d(adm_slots), lazy_n, s)

    def dir_b(self, a_rows, a_k, c_rows, c_cnt, s):
        a_ids, c_slots = self.dx.elara_dir_b(self.stv, self.pv, self._d(a_rows), self._d(a_k), self._d(c_rows), self._d(c_cnt), s)
        assert self.dx.status(self.dev) == 0
        return dict(a_ids=a_ids.cpu().numpy(), c_slots=c_slots.cpu().numpy())

    def state(self):
        return {k: v.cpu().numpy() for k, v in self.t.items()}


@pytest.mark.parametrize('name', ['dir_ttl_evl1', 'dir_ttl_evl0', 'dir_carry_evl1'])
def test_directory_trace_gpu(oracle, golden_dir, name):
    dev = torch.device('cuda:0')
    g = np.load(golden_dir / f'{name}.npz')
    n_rep, n_evl = run_dir_trace(oracle, g, lambda st, pv: GpuDirectory(oracle, st, pv, dev), crc_check(oracle))
    if name.endswith('evl1'):
        assert n_rep > 0 and n_evl > 0


def test_directory_large_random_vs_oracle(oracle):
    """Synthetic calls far larger than the recorded traces (tens of thousands of evictions, appends and compactions per
    call, many CTAs per scan) against the CPU oracle."""
    dev = torch.device('cuda:0')
    rng = np.random.default_rng(11)
    R, K, C, n0, T = 400_000, 3, 120_000, 20_000, 5
    Lcap, Cdyn, MAT = 2 * R, C - n0, K + 1
    pv = dict(R=R, K=K, Lcap=Lcap, n0=n0, Cdyn=Cdyn, MAT=MAT, trash=R, evl=1)
    # a consistent random directory: rows in state L_c own c log entries; resident rows own a slot
    code = rng.choice([0, 1, 2, 3, MAT], size=R, p=[0.4, 0.2, 0.1, 0.1, 0.2]).astype(np.int8)
    ent = np.full((R + 1) * K, -1, np.int32); lstep = np.zeros(Lcap + 1, np.int32)
    top = 0
    for c in (1, 2, 3):
        rows = np.nonzero(code == c)[0]
        for k in range(c):
            ent[rows * K + k] = np.arange(top, top + len(rows)); lstep[top:top + len(rows)] = rng.integers(1, 50, len(rows)); top += len(rows)
    nfree = 30_000
    lfree = np.zeros(Lcap + 1, np.int32); lfree[:nfree] = np.arange(top, top + nfree)[rng.permutation(nfree)]; live = top; top += nfree
    loc = np.full(R + 1, -1, np.int32); mrows = np.nonzero(code == MAT)[0]; loc[mrows] = rng.permutation(len(mrows))
    res_rows = rng.choice(R, C, replace=False)
    slot_of = np.full(R, -1, np.int32); slot_of[res_rows] = np.arange(C); slot_row = res_rows.astype(np.int64)
    adm_c0 = np.where(code[res_rows] == MAT, -1, code[res_rows]).astype(np.int8)
    rj = rng.integers(0, 3, C).astype(np.int8); rok = ((adm_c0 >= 0) & (rng.random(C) < 0.8)).astype(np.int8)
    rj[:n0] = 0; rok[:n0] = 0
    st = dict(code=code, loc=loc, ent=ent, lstep=lstep, lfree=lfree, n_lfree=np.array([nfree]), log_top=np.array([top]),
              mat_top=np.array([len(mrows)]), live=np.array([live]), adm_c0=adm_c0, rj=rj, pstep=rng.integers(1, 50, (Cdyn + 1, K)).astype(np.int32),
              kthr=np.array([3, 2, 3, 1, 3], np.int8), toff=(np.arange(T) * (R // T)).astype(np.int64), slot_of=slot_of, slot_row=slot_row, rok=rok)
    cpu = oracle.Directory({k: v.copy() for k, v in st.items()}, pv)
    gpu = GpuDirectory(oracle, st, pv, dev)
    slots = rng.permutation(C)
    hs, ev_slot = np.sort(slots[:50_000]), slots[30_000:30_000 + 40_000][slots[30_000:70_000] >= n0]
    non_res = np.setdiff1d(np.arange(R), res_rows)
    L_row = non_res[(code[non_res] >= 1) & (code[non_res] <= K)][:30_000]
    L_cnt = code[L_row].astype(np.int32)
    oa, ob = cpu.dir_a(hs, L_row, L_cnt, ev_slot, 60), gpu.dir_a(hs, L_row, L_cnt, ev_slot, 60)
    for k in oa:
        assert np.array_equal(oa[k].reshape(-1).astype(np.int64), ob[k].reshape(-1).astype(np.int64)), k
    assert 0 < oa['rep'].sum() < len(ev_slot)
    adm_rows = non_res[-len(ev_slot):]; lazy = adm_rows[cpu.st['code'][adm_rows] != MAT]; full = adm_rows[cpu.st['code'][adm_rows] == MAT]
    adm_rows = np.concatenate([lazy, full])
    cpu.admit(adm_rows, ev_slot, len(lazy), 60); gpu.admit(adm_rows, ev_slot, len(lazy), 60)
    cand = np.setdiff1d(non_res, adm_rows)
    a_rows = cand[cpu.st['code'][cand] < K][:45_000]; a_k = cpu.st['code'][a_rows].astype(np.int64)
    c_rows = cand[(cpu.st['code'][cand] == K)][:20_000]; c_cnt = np.full(len(c_rows), K, np.int64)
    ra, rb = cpu.dir_b(a_rows, a_k, c_rows, c_cnt, 60), gpu.dir_b(a_rows, a_k, c_rows, c_cnt, 60)
    assert np.array_equal(ra['a_ids'], rb['a_ids']) and np.array_equal(ra['c_slots'], rb['c_slots'])
    assert len(a_rows) > nfree // 2 and len(c_rows) > 1000
    want, got = oracle.dir_comparable(cpu.st, pv), oracle.dir_comparable(gpu.state(), pv)
    for k in oracle.DIR_FIELDS:
        assert np.array_equal(want[k].reshape(-1), got[k].reshape(-1)), k


def test_directory_rejects_bad_indices():
    """Out-of-range slots and rows set the status word; nothing is accessed out of bounds."""
    from elara_b200.ops import dir_ext
    dev = torch.device('cuda:0')
    R, K, C, n0 = 100, 3, 20, 5
    z = lambda n, dt, v=0: torch.full((n,), v, dtype=dt, device=dev)
    st = [z(R, torch.int8), z(R + 1, torch.int32, -1), z((R + 1) * K, torch.int32, -1), z(2 * R + 1, torch.int32), z(2 * R + 1, torch.int32),
          z(1, torch.int64), z(1, torch.int64), z(1, torch.int64), z(1, torch.int64), z(C, torch.int8, -1), z(C, torch.int8),
          torch.zeros(C - n0 + 1, K, dtype=torch.int32, device=dev), z(1, torch.int8, 3), z(1, torch.int64), z(R, torch.int32, -1),
          z(C, torch.int64, -1), z(C, torch.int8)]
    pv = [R, K, 2 * R, n0, C - n0, K + 1, R, 1]
    dx = dir_ext()
    dx.elara_dir_a(st, pv, torch.tensor([1, 999], device=dev), torch.tensor([5, 10_000], device=dev), torch.tensor([1, 1], dtype=torch.int32, device=dev),
                   torch.tensor([-4, 7], device=dev), 1)
    assert dx.status(dev) & 3 == 3
