"""pytest plugin (``-p tests.pathsig_alias_plugin``): makes ``import pathsig`` resolve to this package
before any test module is imported, so that test files written against the reference's public API run
unmodified.  Used by tests/test_gpu_reference_suites.py in a child process of its own (the reference's
own operator library, which other tests load, claims the same ``pathsig`` operator namespace)."""
import pathsig_b200

pathsig_b200.install_as_pathsig()
