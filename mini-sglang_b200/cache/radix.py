"""Prefix cache: a tree over token ids in steps of one page, whose nodes own cache pages.

Semantics follow the reference's radix cache (mini_sglang/mem_cache/radix_cache.py:55-413):
only whole pages are matched; a request pins the path it reads (`lock`/`unlock`, counted from
the node up to the root, :216-238); finished requests donate their full pages and pages that
duplicate tree content are given back (:270-365); when pages are short, unpinned leaves are
evicted least-recently-used first and parents that become leaves follow (:367-405).  The
structure is different: one node per page (the key of an edge is the tuple of the page's
token ids), values are page ids, and eviction returns page ids to the pool that owns them.
"""

from __future__ import annotations

import heapq
import itertools
from typing import Dict, List, Optional, Sequence, Tuple


class Node:
    __slots__ = ("parent", "key", "page", "children", "lock_ref", "last_access", "uid")

    def __init__(self, parent: Optional["Node"], key: Optional[tuple], page: int, uid: int):
        self.parent, self.key, self.page = parent, key, page
        self.children: Dict[tuple, Node] = {}
        self.lock_ref = 0
        self.last_access = 0
        self.uid = uid


class PrefixTree:
    def __init__(self, page_size: int):
        self.page_size = page_size
        self._uid = itertools.count()
        self._clock = itertools.count(1)
        self.root = Node(None, None, 0, next(self._uid))
        self.root.lock_ref = 1                      # the root is never evicted
        self.evictable_pages = 0                    # pages of nodes with lock_ref == 0
        self.protected_pages = 0                    # pages of nodes with lock_ref > 0
        self.num_nodes = 0

    # -- reading -----------------------------------------------------------------------
    def match(self, tokens: Sequence[int]) -> Tuple[List[int], Node]:
        """Longest cached prefix of `tokens` in whole pages -> (page ids, last node)."""
        P = self.page_size
        node, pages = self.root, []
        now = next(self._clock)
        for i in range(len(tokens) // P):
            child = node.children.get(tuple(tokens[i * P:(i + 1) * P]))
            if child is None:
                break
            child.last_access = now
            pages.append(child.page)
            node = child
        return pages, node

    # -- pinning -----------------------------------------------------------------------
    def lock(self, node: Node) -> None:
        """Pin the path from `node` to the root.  A node that was evicted since it was matched is refused:
        its page may belong to someone else by now."""
        up = node
        while up is not self.root:
            if up.parent is None:
                raise RuntimeError("prefix tree: lock of a node that is no longer in the tree (evicted after it was matched)")
            up = up.parent
        while node is not self.root:
            if node.lock_ref == 0:
                self.evictable_pages -= 1
                self.protected_pages += 1
            node.lock_ref += 1
            node = node.parent

    def unlock(self, node: Node) -> None:
        while node is not self.root:
            if node.lock_ref <= 0:
                raise RuntimeError("prefix tree: unlock without lock")
            node.lock_ref -= 1
            if node.lock_ref == 0:
                self.evictable_pages += 1
                self.protected_pages -= 1
            node = node.parent

    # -- writing -----------------------------------------------------------------------
    def insert(self, tokens: Sequence[int], pages: Sequence[int], owned_from: int) -> Tuple[List[int], List[int], Node]:
        """Offer pages[i] for tokens[i*P:(i+1)*P].  Pages with index < owned_from already belong
        to the tree (the request borrowed them).  Returns (table, duplicates, last node): `table`
        is the page list to use from now on (tree pages where the content was already cached),
        `duplicates` are offered pages the tree did not take and the caller must free."""
        P = self.page_size
        n = min(len(tokens) // P, len(pages))
        node, table, dup = self.root, [], []
        now = next(self._clock)
        for i in range(n):
            key = tuple(tokens[i * P:(i + 1) * P])
            child = node.children.get(key)
            if child is None:
                if i < owned_from:
                    raise RuntimeError("prefix tree: a borrowed page is not in the tree")
                child = Node(node, key, pages[i], next(self._uid))
                node.children[key] = child
                self.evictable_pages += 1
                self.num_nodes += 1
            elif i >= owned_from and child.page != pages[i]:
                dup.append(pages[i])
            child.last_access = now
            table.append(child.page)
            node = child
        return table, dup, node

    def evict(self, n_pages: int) -> List[int]:
        """Drop up to n_pages unpinned pages, least recently used leaves first."""
        if n_pages <= 0 or self.evictable_pages == 0:
            return []
        heap = [(nd.last_access, nd.uid, nd) for nd in self._leaves() if nd.lock_ref == 0]
        heapq.heapify(heap)
        freed: List[int] = []
        while heap and len(freed) < n_pages:
            _, _, nd = heapq.heappop(heap)
            if nd.children or nd.lock_ref:
                continue
            freed.append(nd.page)
            parent = nd.parent
            del parent.children[nd.key]
            nd.parent = None                     # detached: lock() refuses it from now on
            self.evictable_pages -= 1
            self.num_nodes -= 1
            if parent is not self.root and not parent.children and parent.lock_ref == 0:
                heapq.heappush(heap, (parent.last_access, parent.uid, parent))
        return freed

    def _leaves(self):
        stack = [self.root]
        while stack:
            nd = stack.pop()
            if nd.children:
                stack.extend(nd.children.values())
            elif nd is not self.root:
                yield nd

    def all_pages(self) -> List[int]:
        out, stack = [], [self.root]
        while stack:
            nd = stack.pop()
            if nd is not self.root:
                out.append(nd.page)
            stack.extend(nd.children.values())
        return out

    def reset(self) -> List[int]:
        """Forget everything (only legal when nothing is pinned) -> the pages that were held."""
        if self.protected_pages:
            raise RuntimeError("prefix tree: reset while pages are pinned")
        pages = self.all_pages()
        stack = list(self.root.children.values())
        while stack:
            nd = stack.pop()
            stack.extend(nd.children.values())
            nd.parent = None
        self.root.children.clear()
        self.evictable_pages = 0
        self.num_nodes = 0
        return pages
