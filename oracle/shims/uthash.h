/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * Stand-in for the hash-table macro header that the ANT-ACE CPU runtime
 * fetches at build time (used in fhe-cmplr/rtlib/ant/include/ckks/key_gen.h
 * and ckks/bootstrap.h).  Only the macros the runtime uses are provided:
 * HASH_FIND_INT, HASH_ADD_INT, HASH_DEL, HASH_ITER, HASH_COUNT.  Elements are
 * kept in an insertion-ordered doubly linked list (iteration order is
 * insertion order, as with the original); look-up is a linear scan, which is
 * ample for the few hundred keys a CKKS context holds.  The container does no
 * arithmetic, so it cannot influence ciphertext values.
 */
#ifndef ORACLE_SHIM_UTHASH_H
#define ORACLE_SHIM_UTHASH_H

#include <stddef.h>

typedef struct UT_hash_handle {
  void*       next;
  void*       prev;
  const void* key;
} UT_hash_handle;

#define UTH_TYPEOF(x) __typeof__(x)

#define HASH_FIND_INT(head, findint, out)                                   \
  do {                                                                      \
    (out) = NULL;                                                           \
    for (UTH_TYPEOF(head) _uth_e = (head); _uth_e != NULL;                  \
         _uth_e                  = (UTH_TYPEOF(head))_uth_e->hh.next) {     \
      if (*(const int*)_uth_e->hh.key == *(const int*)(findint)) {          \
        (out) = _uth_e;                                                     \
        break;                                                              \
      }                                                                     \
    }                                                                       \
  } while (0)

#define HASH_ADD_INT(head, intfield, add)                                   \
  do {                                                                      \
    (add)->hh.key  = &((add)->intfield);                                    \
    (add)->hh.next = NULL;                                                  \
    if ((head) == NULL) {                                                   \
      (add)->hh.prev = NULL;                                                \
      (head)         = (add);                                               \
    } else {                                                                \
      UTH_TYPEOF(head) _uth_t = (head);                                     \
      while (_uth_t->hh.next != NULL)                                       \
        _uth_t = (UTH_TYPEOF(head))_uth_t->hh.next;                         \
      _uth_t->hh.next = (add);                                              \
      (add)->hh.prev  = _uth_t;                                             \
    }                                                                       \
  } while (0)

#define HASH_DEL(head, delptr)                                              \
  do {                                                                      \
    UTH_TYPEOF(head) _uth_d = (delptr);                                     \
    if (_uth_d->hh.prev != NULL)                                            \
      ((UTH_TYPEOF(head))_uth_d->hh.prev)->hh.next = _uth_d->hh.next;       \
    else                                                                    \
      (head) = (UTH_TYPEOF(head))_uth_d->hh.next;                           \
    if (_uth_d->hh.next != NULL)                                            \
      ((UTH_TYPEOF(head))_uth_d->hh.next)->hh.prev = _uth_d->hh.prev;       \
  } while (0)

#define HASH_ITER(hh_name, head, el, tmp)                                   \
  for ((el) = (head),                                                       \
      (tmp) = (UTH_TYPEOF(el))((head) ? (head)->hh_name.next : NULL);       \
       (el) != NULL; (el) = (tmp),                                          \
      (tmp) = (UTH_TYPEOF(el))((tmp) ? (tmp)->hh_name.next : NULL))

#define HASH_COUNT(head)                                                    \
  ({                                                                        \
    unsigned _uth_n = 0;                                                    \
    for (UTH_TYPEOF(head) _uth_c = (head); _uth_c != NULL;                  \
         _uth_c                  = (UTH_TYPEOF(head))_uth_c->hh.next)       \
      _uth_n++;                                                             \
    _uth_n;                                                                 \
  })

#endif /* ORACLE_SHIM_UTHASH_H */
