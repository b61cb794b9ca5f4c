"""Host-side bookkeeping of the cache: pages, slots, and what each sequence holds.

A page holds 64 positions of one storage group. A sequence has a slot (its
row in every per-sequence table) and, in every group, the list of pages that
hold its positions. Pages are handed out when a sequence grows into them and
given back when the sequence ends, or, in a group that keeps only a window,
as soon as every position of the page has left the window. Freed pages and
slots are the next to be handed out again, so reuse happens at once.

The books are kept by the native host runtime (`csrc/host/runtime.cpp`, C
interface in `include/mynah_slm_b200_host.h`); the classes here are its thin
wrappers. Nothing here touches the device; `fill_step` packs the lists into
the tables the kernels read.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Iterator, Optional, Sequence

import numpy as np

class CacheError(RuntimeError):
    pass


_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        from ..csrc.build import host_library_path
        lib = ctypes.CDLL(host_library_path())
        P, I = ctypes.c_void_p, ctypes.c_int
        IP = ctypes.POINTER(ctypes.c_int32)
        lib.mynah_host_last_error.restype = ctypes.c_char_p
        lib.mynah_page_tokens.restype = I
        lib.mynah_page_tokens.argtypes = []
        sigs = {
            "mynah_pool_create": (P, [I]), "mynah_pool_destroy": (None, [P]),
            "mynah_pool_take": (I, [P, I, I, IP]), "mynah_pool_give_back": (I, [P, IP, I, I]),
            "mynah_pool_owner": (I, [P, I]), "mynah_pool_n_free": (I, [P]), "mynah_pool_n_pages": (I, [P]),
            "mynah_slots_create": (P, [I]), "mynah_slots_destroy": (None, [P]), "mynah_slots_take": (I, [P]),
            "mynah_slots_give_back": (I, [P, I]), "mynah_slots_in_use": (I, [P, I]),
            "mynah_slots_n_free": (I, [P]), "mynah_slots_n_slots": (I, [P]),
            "mynah_books_create": (P, [I, IP, I, I]), "mynah_books_destroy": (None, [P]),
            "mynah_books_open": (I, [P]), "mynah_books_close": (I, [P, I]), "mynah_books_length": (I, [P, I]),
            "mynah_books_pages_needed": (I, [P, I, I]), "mynah_books_reserve": (I, [P, I, I]),
            "mynah_books_commit": (I, [P, I, I]), "mynah_books_held": (I, [P, I, I, IP, I, IP]),
            "mynah_books_live_slots": (I, [P, IP, I]), "mynah_books_pool": (P, [P, I]), "mynah_books_slots": (P, [P]),
            "mynah_step_fill": (I, [P, IP, IP, I, I, I, IP, I, IP, IP, IP, IP, IP, IP]),
            "mynah_decode_prepare": (I, [P, I, IP, IP, I, I, IP, IP, I, I, I, IP]),
            "mynah_books_commit_many": (I, [P, I, IP, I]),
            "mynah_randn_fill_host": (I, [P, I, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_ulonglong,
                                          ctypes.c_double, ctypes.c_double]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _LIB = lib
    return _LIB


# Positions a page holds: defined once, in the native runtime's header, and read from the library.
PAGE_TOKENS = int(_lib().mynah_page_tokens())


def host_library():
    """The native host runtime, for the modules that use other parts of it than the cache's books."""
    return _lib()


def _raise() -> None:
    raise CacheError(_lib().mynah_host_last_error().decode(errors="replace"))


def _check(rc: int) -> int:
    if rc < 0:
        _raise()
    return rc


def _ints(values: Sequence[int]):
    return (ctypes.c_int32 * max(len(values), 1))(*values)


class PagePool:
    """Pages 0..n-1 of one group. Tracks the owner of each page so that a
    page can be neither handed out twice nor given back twice."""

    def __init__(self, n_pages: int, _handle=None):
        self._own = _handle is None
        self._h = _handle if _handle is not None else _lib().mynah_pool_create(int(n_pages))
        if not self._h:
            _raise()

    def __del__(self):
        if getattr(self, "_own", False) and self._h and _LIB is not None:
            _LIB.mynah_pool_destroy(self._h)
            self._h = None

    @property
    def n_pages(self) -> int:
        return _lib().mynah_pool_n_pages(self._h)

    @property
    def n_free(self) -> int:
        return _lib().mynah_pool_n_free(self._h)

    def take(self, n: int, owner: int) -> list[int]:
        out = (ctypes.c_int32 * max(n, 1))()
        _check(_lib().mynah_pool_take(self._h, n, owner, out))
        return list(out[:n])

    def give_back(self, pages: list[int], owner: int) -> None:
        _check(_lib().mynah_pool_give_back(self._h, _ints(pages), len(pages), owner))

    def owner(self, page: int) -> Optional[int]:
        o = _lib().mynah_pool_owner(self._h, page)
        if o == -2:
            raise CacheError(f"page {page} does not exist")
        return None if o < 0 else o


class SlotTable:
    def __init__(self, n_slots: int, _handle=None):
        self._own = _handle is None
        self._h = _handle if _handle is not None else _lib().mynah_slots_create(int(n_slots))
        if not self._h:
            _raise()

    def __del__(self):
        if getattr(self, "_own", False) and self._h and _LIB is not None:
            _LIB.mynah_slots_destroy(self._h)
            self._h = None

    @property
    def n_slots(self) -> int:
        return _lib().mynah_slots_n_slots(self._h)

    @property
    def n_free(self) -> int:
        return _lib().mynah_slots_n_free(self._h)

    def take(self) -> int:
        return _check(_lib().mynah_slots_take(self._h))

    def give_back(self, slot: int) -> None:
        _check(_lib().mynah_slots_give_back(self._h, slot))

    def in_use(self, slot: int) -> bool:
        return bool(_lib().mynah_slots_in_use(self._h, slot))


@dataclass
class GroupPlan:
    """Storage group: the cache entries (runs of layers) that need the same
    thing per position and may therefore share page lists."""
    kv_heads: int
    head_dim: int
    window: Optional[int]          # None: every position is kept
    entries: list[int] = field(default_factory=list)    # schedule indices stored here
    v_head_dim: Optional[int] = None                     # width of the values; None: head_dim; 0: keys only


class _Lengths:
    """`length[slot]`, `slot in length`, iteration over the live slots: a read-only view of the books."""

    def __init__(self, books: "SequencePages"):
        self._b = books

    def __getitem__(self, slot: int) -> int:
        n = _lib().mynah_books_length(self._b._h, int(slot))
        if n < 0:
            raise KeyError(slot)
        return n

    def __contains__(self, slot) -> bool:
        return _lib().mynah_books_length(self._b._h, int(slot)) >= 0

    def __iter__(self) -> Iterator[int]:
        return iter(self._b.live_slots())

    def __len__(self) -> int:
        return _lib().mynah_books_live_slots(self._b._h, None, 0)


class SequencePages:
    """What the live sequences hold, in every group."""

    def __init__(self, groups: list[GroupPlan], n_pages: int, max_seqs: int):
        self.groups = groups
        windows = _ints([int(g.window) if g.window is not None else 0 for g in groups])
        self._h = _lib().mynah_books_create(len(groups), windows, int(n_pages), int(max_seqs))
        if not self._h:
            _raise()
        self.pools = [PagePool(0, _handle=_lib().mynah_books_pool(self._h, g)) for g in range(len(groups))]
        self.slots = SlotTable(0, _handle=_lib().mynah_books_slots(self._h))
        self.length = _Lengths(self)
        self._n_pages = int(n_pages)

    def __del__(self):
        if getattr(self, "_h", None) and _LIB is not None:
            _LIB.mynah_books_destroy(self._h)
            self._h = None

    # ---------------------------------------------------------- lifecycle
    def open(self) -> int:
        return _check(_lib().mynah_books_open(self._h))

    def close(self, slot: int) -> None:
        _check(_lib().mynah_books_close(self._h, int(slot)))

    # -------------------------------------------------------------- growth
    def pages_needed(self, slot: int, n_new: int) -> int:
        """Pages the fullest group still has to take for n_new more positions."""
        return _check(_lib().mynah_books_pages_needed(self._h, int(slot), int(n_new)))

    def reserve(self, slot: int, n_new: int) -> None:
        """Make sure every position below length + n_new has a page in every group."""
        _check(_lib().mynah_books_reserve(self._h, int(slot), int(n_new)))

    def commit(self, slot: int, n_new: int) -> None:
        """The positions have been written: advance, and let windowed groups
        give back the pages no later query can see."""
        _check(_lib().mynah_books_commit(self._h, int(slot), int(n_new)))

    # --------------------------------------------------------------- views
    def held(self, slot: int, group: int) -> tuple[list[int], int]:
        base = ctypes.c_int32(0)
        n = _check(_lib().mynah_books_held(self._h, int(slot), int(group), None, 0, ctypes.byref(base)))
        out = (ctypes.c_int32 * max(n, 1))()
        _check(_lib().mynah_books_held(self._h, int(slot), int(group), out, n, ctypes.byref(base)))
        return list(out[:n]), int(base.value)

    def n_held(self, slot: int, group: int) -> int:
        return _check(_lib().mynah_books_held(self._h, int(slot), int(group), None, 0, None))

    def live_slots(self) -> list[int]:
        n = _lib().mynah_books_live_slots(self._h, None, 0)
        out = (ctypes.c_int32 * max(n, 1))()
        _lib().mynah_books_live_slots(self._h, out, n)
        return list(out[:n])

    # ------------------------------------------------- the step's description
    def fill_step(self, buf: np.ndarray, offsets: np.ndarray, T: int, B: int, W: int, ids_cap: np.ndarray,
                  slots: Sequence[int], token_lists: Sequence[Sequence[int]],
                  want_lists: Optional[Sequence[Sequence[int]]]) -> tuple[int, int]:
        """Packs a step's batch description into `buf` (int32, the layout whose field offsets are `offsets`).
        Returns (longest entry, wanted rows)."""
        n = len(slots)
        ip = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
        slot_a = np.asarray(slots, dtype=np.int32)
        n_tok = np.fromiter((len(t) for t in token_lists), dtype=np.int32, count=n)
        arrays = [np.asarray(t, dtype=np.int32) for t in token_lists]
        toks = arrays[0] if n == 1 else (np.concatenate(arrays) if n else np.zeros((0,), dtype=np.int32))
        toks = np.ascontiguousarray(toks)
        if want_lists is not None:
            n_want = np.fromiter((len(w) for w in want_lists), dtype=np.int32, count=n)
            want = np.fromiter((int(x) for w in want_lists for x in w), dtype=np.int32, count=int(n_want.sum()))
            nw_p, w_p = ip(n_want), ip(want) if want.size else None
        else:
            nw_p = w_p = None
        rows = ctypes.c_int32(0)
        max_q = _check(_lib().mynah_step_fill(self._h, ip(buf), ip(offsets), T, B, W, ip(ids_cap), n, ip(slot_a), ip(n_tok),
                                              ip(toks) if toks.size else None, nw_p, w_p, ctypes.byref(rows)))
        return max_q, int(rows.value)

    def max_length(self, slots: Sequence[int]) -> int:
        return max(self.length[s] for s in slots)

    def decode_prepare(self, buf: np.ndarray, offsets: np.ndarray, T: int, B: int, W: int, ids_cap: np.ndarray,
                       slots: np.ndarray, tokens: np.ndarray, vocab: int, max_positions: int) -> int:
        """One more token for each of `slots` (int32 arrays): checks, pages and the step's description in one
        native call. Returns the longest sequence after the step."""
        ip = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
        return _check(_lib().mynah_decode_prepare(self._h, len(slots), ip(slots), ip(tokens), int(vocab), int(max_positions),
                                                  ip(buf), ip(offsets), T, B, W, ip(ids_cap)))

    def commit_many(self, slots: np.ndarray, n_new: int) -> None:
        _check(_lib().mynah_books_commit_many(self._h, len(slots), slots.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(n_new)))
