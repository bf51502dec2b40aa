"""L8 trainer runtime: environment, assembly, engine, gradient / batch / metric services, observer."""
