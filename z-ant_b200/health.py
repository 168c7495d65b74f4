"""Per-rank status exchange for the multi-process (one process per GPU) form of sample sharding.

Samples are independent, so the ranks of a sharded predict never wait for one another on the GPU; the only place
a rank can hang is a host-side barrier or reduction that a failed peer never joins.  Each rank therefore publishes
a status code per step in a key-value store (any object with torch.distributed.Store's `set` / `get` / `wait`), and
looks at its peers' codes before it enters a collective: a peer that reported a failure, or that did not report
within the timeout, is named in the per-rank status array instead of being waited for.  The codes are the
library's zant_status values (0 = OK); -1000 stands for "no report".
"""
import datetime

NO_REPORT = -1000


class RankHealth:
    def __init__(self, store, rank, world, timeout_s=10.0):
        self.store, self.rank, self.world = store, rank, world
        self.timeout = datetime.timedelta(seconds=timeout_s)

    def _key(self, rank, step):
        return f"zant_b200/status/{step}/{rank}"

    def report(self, step, status=0):
        """Publishes this rank's status for `step` (call it between steps, with no kernel or collective in flight)."""
        self.store.set(self._key(self.rank, step), str(int(status)))

    def statuses(self, step):
        """Status of every rank for `step`; ranks that do not report within the timeout get NO_REPORT."""
        out = []
        for r in range(self.world):
            try:
                self.store.wait([self._key(r, step)], self.timeout)
                out.append(int(self.store.get(self._key(r, step)).decode()))
            except Exception:       # noqa: BLE001  (the store raises a plain RuntimeError / DistStoreError on timeout)
                out.append(NO_REPORT)
        return out

    def all_ok(self, step):
        s = self.statuses(step)
        return all(v == 0 for v in s), s
