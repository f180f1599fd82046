"""Drop-in module names for users coming from the reference project.

The reference is a flat set of modules (``utils``, ``baseline``, ``layers.all_to_all``,
``layers.token_shuffle``, ``layers.expert``).  The sub-modules here carry the same names and
export the same call signatures, implemented by this package:

    from iris_testing_b200.compat.utils import gen_local_tokens, route_and_pack_padding_free
    from iris_testing_b200.compat.layers.all_to_all import custom_a2a
    from iris_testing_b200.compat.baseline import run_baseline_ref, init_baseline_buffers
"""
