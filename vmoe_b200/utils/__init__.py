"""General helpers: call-string parsing, partial classes, safe zips, regex matchers, RNG streams.

Behavioural counterpart of the reference's ``vmoe/utils.py``.
"""
from vmoe_b200.utils.misc import (SafeZipIterator, SafeZipIteratorError, make_match_fn_from_regex_list,
                                  make_rngs, multiply_no_nan, parse_call, partialclass, safe_map,
                                  safe_zip, tree_rngs_split, flatten_dict, unflatten_dict,
                                  natural_sort_key)
from vmoe_b200.utils.config_dict import ConfigDict, FieldReference, FrozenConfigDict, placeholder
