"""Context parallelism: Ulysses all-to-all (``ulysses``), ring attention (``ring``), sequence split/gather
helpers and zig-zag load balancing (``split``)."""
