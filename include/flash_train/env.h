/*
 * flash_train/env.h -- names of the environment variables the library reads.
 *
 * Same four variables, same meaning, as the reference
 * (include/flash_train/env.h:24-48). Every variable is read once, the first
 * time the library needs it. A name list is split at commas and each entry is
 * stripped of surrounding spaces and tabs. A switch is ON when its stripped
 * value is non-empty and is not "0".
 */
#ifndef FTRAIN_ENV_H_
#define FTRAIN_ENV_H_

/* Allowlist of Primitive names: when set, only listed Primitives are selected. */
#define FTRAIN_ENABLED_PRIMITIVES "FTRAIN_ENABLED_PRIMITIVES"

/* Denylist of Primitive names: listed Primitives are never selected. */
#define FTRAIN_DISABLED_PRIMITIVES "FTRAIN_DISABLED_PRIMITIVES"

/* Denylist of Finder names: listed Finders contribute no candidates. */
#define FTRAIN_DISABLED_FINDERS "FTRAIN_DISABLED_FINDERS"

/* Switch: bypass the selection cache, re-running selection on every Plan. */
#define FTRAIN_DISABLE_CACHE "FTRAIN_DISABLE_CACHE"

#endif
