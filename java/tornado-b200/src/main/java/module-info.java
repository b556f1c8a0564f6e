module tornado.b200 {
    requires transitive tornado.api;
    requires tornado.runtime;

    exports uk.ac.manchester.tornado.b200;

    provides uk.ac.manchester.tornado.runtime.library.spi.TornadoLibraryProvider
            with uk.ac.manchester.tornado.b200.provider.B200LibraryProvider;
}
