"""Reference import names (``communication.*``) as thin aliases of :mod:`conef_b200.parallel`."""
