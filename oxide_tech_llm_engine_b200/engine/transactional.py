"""Transactional block-table updates: make room for tokens, then either commit or roll back.

`with KvTransaction(table, n_tokens) as tx:` reserves the blocks; leaving the block without
`tx.commit()` (an exception, an early return) returns them to the pool and restores the committed
length, like the reference's `TransactionalKvGuard` whose drop rolls back
(crates/oxide-alloc/src/transactional.rs:77-128). `table` is the C++ `SequenceBlockTable`.
"""
from __future__ import annotations

from ..errors import OutOfMemory, TransactionAborted


class KvTransaction:
    def __init__(self, table, n_tokens: int):
        self.table, self.n = table, int(n_tokens)
        self.cow: list = []
        self._done = False

    def __enter__(self) -> "KvTransaction":
        ok, cow = self.table.advance(self.n)
        if not ok:
            raise OutOfMemory(f"no room for {self.n} more tokens")
        self.cow = list(cow)
        return self

    def commit(self) -> None:
        self.table.commit()
        self._done = True

    def abort(self, why: str = "aborted") -> None:
        self.table.rollback()
        self._done = True
        raise TransactionAborted(why)

    def __exit__(self, et, ev, tb) -> bool:
        if not self._done:
            self.table.rollback()
            self._done = True
        return False
